"""Ownership arithmetic of the all-gather GEMM (``window_ownership`` / ``remote_chunks_in_block``
/ the copy role's chunk walk in ``csrc/kernels/gemm2_kernel.cuh``) restated on the host and
checked over random placements: the weight is a window of a flat buffer that the ranks shard in
contiguous 8 KiB-aligned pieces, so ownership boundaries fall anywhere inside the matrix and
some ranks own nothing of it.  Every remote chunk must be copied exactly once, by its owner's
pointer, never the rank's own chunks, and the per-block counts the TMA producers wait for must
equal what the copy warps will announce - a mismatch there is a GEMM that waits out its budget."""
import random

CHUNK = 8192


def ownership(world, rank, w_off, w_bytes, shard):
    n_total = -(-w_bytes // CHUNK)
    lo = min(max(rank * shard - w_off, 0), w_bytes)
    hi = min(max((rank + 1) * shard - w_off, 0), w_bytes)
    oc_lo, oc_hi = lo // CHUNK, -(-hi // CHUNK)
    if hi <= lo:
        oc_lo = oc_hi = 0
    start = oc_hi % n_total if oc_hi > oc_lo else (rank * n_total) // world
    return n_total, oc_lo, oc_hi, start


def remote_chunks_in_block(nb, block_bytes, n_total, oc_lo, oc_hi):
    per = block_bytes // CHUNK
    c0, c1 = nb * per, min(nb * per + per, n_total)
    if c1 <= c0:
        return 0
    a, b = max(c0, oc_lo), min(c1, oc_hi)
    return (c1 - c0) - (b - a if b > a else 0)


def test_every_remote_chunk_once_and_block_counts_agree():
    rng = random.Random(0)
    for _ in range(4000):
        world = rng.choice([2, 3, 4, 8])
        k = rng.choice([64, 128, 256, 512, 5120, 8192])
        n = rng.randint(1, 40) * rng.choice([8, 64, 100, 256])
        w_bytes, w_off = n * k * 2, rng.randint(0, 50) * CHUNK
        total = w_off + w_bytes + rng.randint(0, 30) * CHUNK
        shard = -(-total // (world * CHUNK)) * CHUNK
        block_bytes, nt = 256 * k * 2, -(-n // 256)
        for rank in range(world):
            n_total, oc_lo, oc_hi, start = ownership(world, rank, w_off, w_bytes, shard)
            n_remote = n_total - (oc_hi - oc_lo)
            copiers = rng.choice([2, 12, 148])
            seen = {}
            for cta in range(copiers):
                mine = (n_remote - cta + copiers - 1) // copiers if n_remote > cta else 0
                for q in range(mine):
                    c = (start + cta + q * copiers) % n_total
                    off = c * CHUNK
                    owner = (w_off + off) // shard
                    assert 0 <= owner < world and owner != rank
                    last = min(off + CHUNK, w_bytes) - 1
                    assert (w_off + last) // shard == owner          # a chunk never straddles two owners
                    seen[c] = seen.get(c, 0) + 1
            assert len(seen) == n_remote and all(v == 1 for v in seen.values())
            for c in range(oc_lo, oc_hi):                              # what is skipped really is this rank's
                assert (w_off + c * CHUNK) // shard == rank
            announced = {}
            for c in seen:
                announced[(c * CHUNK) // block_bytes] = announced.get((c * CHUNK) // block_bytes, 0) + 1
            for nb in range(nt):
                assert announced.get(nb, 0) == remote_chunks_in_block(nb, block_bytes, n_total, oc_lo, oc_hi)


def test_row_sharded_matrix_is_the_special_case():
    """w_off = 0 and shard = rows/world * row bytes: rank r owns exactly its rows' chunks."""
    world, n, k = 4, 4096, 2048
    shard = n // world * k * 2
    for rank in range(world):
        n_total, oc_lo, oc_hi, start = ownership(world, rank, 0, n * k * 2, shard)
        assert (oc_lo, oc_hi) == (rank * shard // CHUNK, (rank + 1) * shard // CHUNK)
        assert start == oc_hi % n_total
