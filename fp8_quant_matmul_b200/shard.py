"""N-partition of one GEMM over several GPUs (one process per GPU).

Every column block of C depends only on the matching rows of B / b_scale and on all of A /
a_scale (check.cu:42-48), so the partition needs no exchange on the GEMM path: A and a_scale
are replicated, rank g owns a contiguous column range of B and writes its own M x N_local
slab of C.  The reference has no multi-GPU code; this is the new build's only parallel mode.
"""
import numpy as np

GRANULE = 64   # shard boundaries fall on multiples of 64 columns (16-byte TMA strides need N_local % 16 == 0)


def plan_n_shards(N, world_size, granule=GRANULE):
    """[(n0, n_local)] for ranks 0..world_size-1: contiguous, covering [0, N), boundaries on `granule`.

    Slabs of `granule` columns are dealt as evenly as possible (the first ranks get one more);
    a ragged tail shorter than a granule goes to the last rank that owns any column.  Ranks
    beyond the number of slabs get (N, 0).
    """
    if N <= 0 or world_size <= 0:
        raise ValueError("N and world_size must be positive")
    slabs = max(1, N // granule)
    base, extra = divmod(slabs, world_size)
    counts = [base + (1 if r < extra else 0) for r in range(world_size)]
    last_owner = max(r for r in range(world_size) if counts[r])
    out, n0 = [], 0
    for r in range(world_size):
        if counts[r] == 0:
            out.append((N, 0))
            continue
        n1 = N if r == last_owner else n0 + counts[r] * granule
        out.append((n0, n1 - n0))
        n0 = n1
    assert sum(c for _, c in out) == N, (N, world_size, out)
    return out


def shard_columns_of_B(B, N, K, n0, n_local):
    """Re-pack columns [n0, n0+n_local) of a column-major N x K byte matrix as a contiguous
    n_local x K column-major matrix (what rank g passes as B)."""
    Bm = np.asarray(B).reshape(K, N)
    return np.ascontiguousarray(Bm[:, n0:n0 + n_local]).ravel()


def gather_columns_of_C(slabs, plan, M, N):
    """Row-major M x N from per-rank M x n_local slabs (the host-side view of the all-gather)."""
    out = np.empty((M, N), dtype=np.asarray(slabs[0]).dtype)
    for slab, (n0, n_local) in zip(slabs, plan):
        if n_local:
            out[:, n0:n0 + n_local] = np.asarray(slab).reshape(M, n_local)
    return out
