"""Example solution for the op `allreduce`: one launch on the symmetric heap instead of an NCCL call.

`rc.comm.all_reduce` stages the input into memory every rank maps, crosses an in-kernel barrier and reduces with direct
peer loads (or the no-barrier exchange for small messages, or the in-switch form for large ones); nothing returns to the
host. On CPU ranks the same call runs on the shared-memory twin, so the file can be evaluated without a GPU."""


def solution(rc, x):
    return rc.comm.all_reduce(x)
