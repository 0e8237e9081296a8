"""Index arithmetic of the peer-gather copy role (``gather_role`` in
``csrc/kernels/gemm_kernel.cuh``), restated on the host: for every world size,
copier count and shard size in use, the chunks handed to the copier CTAs must
cover every remote shard exactly once, in pieces the bulk-copy instructions
accept (16-byte aligned, multiples of 16 bytes), and the per-block ready
counters must stay inside their array."""
import pytest

CHUNK = 8192            # PG_CHUNK of ft_peer_gather
READY_WORDS = 8192      # kReadyWords


def _walk(world, rank, shard_bytes, copiers, block_bytes):
    chunks_per_shard = (shard_bytes + CHUNK - 1) // CHUNK
    total = chunks_per_shard * (world - 1)
    covered, max_block = {}, 0
    for cta in range(copiers):
        n = (total - cta + copiers - 1) // copiers if total > cta else 0
        for q in range(n):
            gq = cta + q * copiers
            k = gq // chunks_per_shard
            peer = (rank + 1 + k) % world
            in_shard = (gq % chunks_per_shard) * CHUNK
            off = peer * shard_bytes + in_shard
            nbytes = min(shard_bytes - in_shard, CHUNK)
            assert peer != rank and 0 <= k < world - 1
            assert off % 16 == 0 and nbytes % 16 == 0 and nbytes > 0
            covered.setdefault(peer, []).append((in_shard, nbytes))
            max_block = max(max_block, off // block_bytes)
    return covered, max_block


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("shard_elems", [106956800, 158603264, 99328 * 2, 8 * 4099])   # 70B/8, 13B/2, tiny
@pytest.mark.parametrize("copiers", [16, 64, 148])
def test_chunks_cover_every_remote_shard_once(world, shard_elems, copiers):
    shard_bytes = shard_elems * 2
    block_bytes = max((shard_bytes * world + READY_WORDS - 1) // READY_WORDS, CHUNK)
    for rank in (0, world - 1):
        covered, max_block = _walk(world, rank, shard_bytes, copiers, block_bytes)
        assert sorted(covered) == [p for p in range(world) if p != rank]
        for pieces in covered.values():
            pieces.sort()
            pos = 0
            for start, n in pieces:
                assert start == pos
                pos += n
            assert pos == shard_bytes
        assert max_block < READY_WORDS
