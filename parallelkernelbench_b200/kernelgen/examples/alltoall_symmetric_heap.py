"""Example solution for the op `alltoall`: the input is [W, m, n] and chunk g of every rank goes to rank g.

`rc.comm.all_to_all` does the exchange in one launch: the input is staged into memory every rank maps, an in-kernel barrier
publishes it, and every rank pulls its chunk from every peer with 16-byte loads over NVLink (large chunks as TMA bulk
requests) - no split-size lists and no host synchronisation."""


def solution(rc, x):
    if rc.world == 1:
        return x.clone()
    return rc.comm.all_to_all(x.contiguous())
