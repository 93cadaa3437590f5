"""Host-side logic for running the sampler on several GPUs of one node (one process per GPU).

Batch sharding: rows are independent (one cluster per row, one RNG state per row), so rank r
takes a contiguous slice of rows, with NO collective on the data path.  The RNG subsequence of
a row is its GLOBAL row index, so a sharded run draws exactly the numbers of the unsharded run
(the reference seeds row b with subsequence b, sampling.cu:137).
"""
import ctypes as C


def row_range(B, rank, world):
    """Contiguous, balanced slice [start, stop) of B rows for `rank` of `world` (first ranks get the remainder)."""
    if not (0 <= rank < world) or B < 0:
        raise ValueError("bad shard request B=%d rank=%d world=%d" % (B, rank, world))
    base, rem = divmod(B, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def vocab_range(V, rank, world):
    """Column slice of a vocab-parallel shard: V/world columns, which must stay a multiple of 4."""
    if V % world or (V // world) % 4:
        raise ValueError("V=%d cannot be split into %d shards of a multiple of 4 columns" % (V, world))
    w = V // world
    return rank * w, (rank + 1) * w


def setup_rand_rows(seed, first_row, n_rows, device=None):
    """RNG states for global rows [first_row, first_row + n_rows) on the current CUDA device: int8[n_rows*64]."""
    import torch
    from . import abi
    L = abi.load()
    st = torch.empty(n_rows * abi.RS_STATE_BYTES, dtype=torch.int8, device=device or "cuda")
    rc = L.rs_setup_rand(st.data_ptr(), seed & (2 ** 64 - 1), n_rows, first_row,
                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(abi.status_string(rc))
    return st
