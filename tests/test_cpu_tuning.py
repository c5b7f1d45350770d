"""Algorithm selection table: the packaged thresholds, overrides by file, and the rule that turns measured timings into a row."""
import json

from parallelkernelbench_b200 import tuning


def test_packaged_table_selects_by_size_and_world():
    K, M = 1024, 1024 * 1024
    pick = lambda n, w, ll=True, nvls=True: tuning.all_reduce_algo(n, w, ll_ok=ll, nvls_ok=nvls)  # noqa: E731
    assert pick(4 * K, 2) == "ll" and pick(256 * K, 8) == "ll"
    assert pick(4 * K, 2, ll=False) == "oneshot"                       # dtype or op the exchange does not take
    assert pick(16 * M, 2) == "oneshot" and pick(128 * M, 2) == "twoshot"      # two ranks: a peer read costs what the switch costs
    assert pick(1 * M, 8) == "nvls" and pick(1 * M, 8, nvls=False) == "twoshot"
    assert pick(512 * K, 4) == "oneshot" and pick(512 * K + 2, 4) == "nvls"
    assert pick(128 * M, 3) == "twoshot"
    assert pick(1 << 30, 1) == "oneshot"
    assert tuning.all_gather_ll_max(8) == 256 * K


def test_table_file_override_and_version_check(tmp_path, monkeypatch):
    p = tmp_path / "t.json"
    p.write_text(json.dumps({"version": 1, "all_reduce": {"default": {"ll_max_bytes": 0, "oneshot_max_bytes": 64, "large": "twoshot"}}}))
    t = tuning.load_table(str(p))
    assert tuning.all_reduce_algo(32, 4, ll_ok=True, nvls_ok=True, table=t) == "oneshot"
    assert tuning.all_reduce_algo(128, 4, ll_ok=True, nvls_ok=True, table=t) == "twoshot"
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"version": 7}))
    try:
        tuning.load_table(str(bad))
    except ValueError as e:
        assert "version" in str(e)
    else:
        raise AssertionError("a table of an unknown version must be rejected")


def test_thresholds_from_timings_finds_the_crossovers():
    t = {"ll": {4096: 6.7, 65536: 9.0, 1048576: 23.6},
         "oneshot": {4096: 11.0, 65536: 12.0, 1048576: 15.0, 16777216: 52.0, 134217728: 600.0},
         "twoshot": {4096: 20.0, 65536: 21.0, 1048576: 25.0, 16777216: 60.0, 134217728: 261.0},
         "nvls": {4096: 22.0, 65536: 22.0, 1048576: 26.0, 16777216: 70.0, 134217728: 429.0}}
    row = tuning.thresholds_from_timings(t)
    assert row == {"ll_max_bytes": 65536, "oneshot_max_bytes": 16777216, "large": "twoshot"}
    t["nvls"][134217728] = 200.0
    assert tuning.thresholds_from_timings(t)["large"] == "nvls"


def test_push_and_in_switch_thresholds_come_from_the_table():
    """All-gather / reduce-scatter / broadcast in-switch thresholds and the all-to-all push thresholds are table rows too: absent
    rows mean "never", the all-to-all has a separate (lower) threshold for results that already live in the symmetric heap."""
    t = {"version": 1, "all_gather": {"4": {"ll_max_bytes": 1024, "nvls_min_bytes": 4096}}, "reduce_scatter": {"8": {"nvls_min_bytes": 8192}},
         "broadcast": {"default": {"nvls_min_bytes": 2048}},
         "all_to_all": {"default": {"push_min_bytes": 1 << 23, "push_direct_min_bytes": 1 << 20}}}
    assert tuning.all_gather_nvls_min(4, t) == 4096 and tuning.all_gather_nvls_min(2, t) > 1 << 60
    assert tuning.reduce_scatter_nvls_min(8, t) == 8192 and tuning.reduce_scatter_nvls_min(4, t) > 1 << 60
    assert tuning.broadcast_nvls_min(3, t) == 2048
    assert tuning.all_to_all_push_min(4, t) == 1 << 23 and tuning.all_to_all_push_min(4, t, direct=True) == 1 << 20
    # the committed table parses and keeps the orderings the kernels rely on
    assert tuning.all_to_all_push_min(4, direct=True) <= tuning.all_to_all_push_min(4)
    assert tuning.all_gather_nvls_min(8) >= tuning.all_gather_ll_max(8)
