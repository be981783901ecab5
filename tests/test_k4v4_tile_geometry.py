"""CPU model of how the K4V4 scan cuts a row into two-page tiles when the weights follow the
reference's batch > 1 Stage B: the host's tile table and the kernel's per-tile arithmetic
(``launch_scan_k4v4`` / ``tile_geom`` in jetfire_b200/csrc/decode_scan_k4v4.cu, restated here
line for line) must produce exactly the tiles of the oracle's loop -- 8 splits of
ceil(max_S / 8) positions, 32-token tiles from each split's first 16-token block
(jetfire_vllm/csrc/int8tc_softmax_v_fused.cu:62, 1049-1053 of JetFire) -- for every max_S and
length, including splits that cut a block in two, and tiles past a row's own length must form
a suffix of the tile order (the kernel stops at the first one)."""
import pytest


def host_tiles(max_S):
    chunk = (max_S + 7) // 8
    base, n = [], 0
    for s in range(8):
        base.append(n)
        lo, hi = s * chunk, min(s * chunk + chunk, max_S)
        if lo < hi:
            n += ((hi + 15) // 16 - lo // 16 + 1) // 2
    base.append(n)
    return chunk, base, n


def device_tile(gT, chunk, base, n_tiles, length):
    if gT >= n_tiles:
        return None
    s, b = 0, 0
    for i in range(1, 8):
        if gT >= base[i]:
            s, b = i, base[i]
    s_lo, s_hi = s * chunk, min(s * chunk + chunk, length)
    page_a = (s_lo >> 4) + 2 * (gT - b)
    blk_end = (s_hi + 15) >> 4
    if s_lo >= s_hi or page_a >= blk_end:
        return None
    pa, two = page_a * 16, page_a + 1 < blk_end
    lo_a, hi_a = max(s_lo - pa, 0), min(s_hi - pa, 16)
    hi_b = min(s_hi - pa - 16, 16) if two else 0
    assert 0 <= lo_a < hi_a <= 16 and 0 <= hi_b <= 16
    return set(range(pa + lo_a, pa + hi_a)) | set(range(pa + 16, pa + 16 + hi_b))


def oracle_tiles(max_S, n):
    chunk, out = (max_S + 7) // 8, []
    for sp in range(8):
        lo, hi = sp * chunk, min((sp + 1) * chunk, n)
        t0 = (lo // 16) * 16
        while lo < hi and t0 < hi:
            a, b = max(t0, lo), min(t0 + 32, hi)
            if a < b:
                out.append(set(range(a, b)))
            t0 += 32
    return out


@pytest.mark.parametrize("max_S", list(range(1, 300)) + [1000, 1008, 4096, 32768, 33000, 40000, 262144])
def test_tiles_match_the_reference_layout(max_S):
    chunk, base, n_tiles = host_tiles(max_S)
    for length in sorted({0, 1, 17, max_S // 3, max_S // 2, max_S - 13, max_S - 1, max_S}):
        if not 0 <= length <= max_S:
            continue
        tiles, dead = [], False
        for gT in range(n_tiles):
            t = device_tile(gT, chunk, base, n_tiles, length)
            if t is None:
                dead = True
                continue
            assert not dead, "a live tile after a dead one"
            tiles.append(t)
        assert tiles == oracle_tiles(max_S, length)
