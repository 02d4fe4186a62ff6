"""Tensor-parallel plumbing: one process per GPU, torch.distributed only swaps the
64-byte CUDA IPC handles of the ranks' exchange buffers; the data path is the decode
kernel's own peer stores over NVLink (no collective library call per token)."""


def connect(model, dist, rank, world):
    """Exchange IPC handles over the process group and connect `model`'s ranks."""
    dist.barrier()  # no rank may still run a step when the buffers are (re)connected and cleared
    mine = model.tp_export()
    handles = [None] * world
    dist.all_gather_object(handles, mine)
    model.tp_connect(handles)
    dist.barrier()
    return handles


def shard_rows(n_rows, rank, world):
    """Row window [r0, r0+nr) of a row-split weight (QKV, gate, up, output)."""
    nr = n_rows // world
    return rank * nr, nr


def shard_cols(n_cols, rank, world):
    """Column window of a column-split weight (o_proj, down): whole 32-column blocks."""
    nc = n_cols // world
    assert nc % 32 == 0, "column shards must be whole Q8_0 blocks"
    return rank * nc, nc


def slice_q8_0(blocks34, rows, cols, r0, nr, c0, nc):
    """Cut the [r0:r0+nr, c0:c0+nc] window out of a [rows, cols] matrix of 34-byte blocks."""
    import numpy as np
    b = np.asarray(blocks34, np.uint8).reshape(rows, cols // 32, 34)
    return np.ascontiguousarray(b[r0:r0 + nr, c0 // 32:(c0 + nc) // 32]).reshape(-1)
