"""Pure-integer models of the kernels' address arithmetic (no GPU): each restates an index
formula of a kernel source file and checks the property the kernel relies on, the way the
reference checks its grid swizzle and ldmatrix bank mapping with integer models
(src/ptx_emitter.rs:7449-7513, 8265-8365)."""
import itertools

import pytest


def _banks(byte_addr: int, nbytes: int):
    return [((byte_addr + 4 * i) // 4) % 32 for i in range(nbytes // 4)]


@pytest.mark.parametrize("head_dim", [64, 128, 256])
def test_attention_staging_swizzle_is_conflict_free_for_ldmatrix(head_dim):
    """attention.cu: K/V rows of head_dim f16 sit row_bytes apart; the 16-byte chunk c of row r
    is stored at chunk c ^ (r & 7). Every 8x8 block one ldmatrix phase reads (8 consecutive
    rows, one logical chunk) must touch each of the 32 banks exactly once, for K (plain) and
    V (transposed) alike, and the mapping must be a permutation of the row's chunks."""
    row_bytes, chunks = head_dim * 2, head_dim // 8
    for r in range(16):
        assert sorted(c ^ (r & 7) for c in range(chunks)) == list(range(chunks))
    for r0 in (0, 8):
        for c in range(chunks):
            hit = []
            for r in range(r0, r0 + 8):
                hit += _banks(r * row_bytes + ((c ^ (r & 7)) * 16), 16)
            assert sorted(hit) == list(range(32))


def test_transposed_quantise_tile_swizzle():
    """quantize.cu: thread t = 8*rq + cv (rq 0..31, cv 0..7) stores, for j in 0..7, the word
    of column cv*8+j at word index rq ^ (cv*4) of that column's 32-word row; a warp's 32
    stores of one j must hit 32 different banks. The write-out reads 16-byte groups
    (rv ^ (c // 8)) * 4 of row c: together they must return every row quad once."""
    for warp in range(8):
        for j in range(8):
            banks = set()
            for lane in range(32):
                t = warp * 32 + lane
                rq, cv = t // 8, t % 8
                word = (cv * 8 + j) * 32 + (rq ^ (cv * 4))
                banks.add(word % 32)
            assert len(banks) == 32
    for c in range(64):
        cv = c // 8
        stored = {rq: rq ^ (cv * 4) for rq in range(32)}           # row quad -> word index
        read_back = {}
        for rv in range(8):
            g = (rv ^ cv) * 4
            for i in range(4):
                read_back[g + i] = rv * 4 + i                       # word index -> row quad it is taken for
        assert all(read_back[w] == rq for rq, w in stored.items())


@pytest.mark.parametrize("head_dim", [64, 128, 256])
def test_rope_span_mapping_covers_every_pair_once(head_dim):
    """quantize.cu rope_kernel: a warp works on a span of 128 pairs; lane L takes pairs
    [4L, 4L+3] of the span: row (4L) // pairs_per_row of the span, pair (4L) % pairs_per_row."""
    ppr = head_dim // 2
    rows_per_span = 128 // ppr
    seen = set()
    for lane in range(32):
        row, p0 = (lane * 4) // ppr, (lane * 4) % ppr
        assert row < rows_per_span and p0 + 3 < ppr
        for j in range(4):
            seen.add((row, p0 + j))
    assert len(seen) == 128 == rows_per_span * ppr


def _pair_units(tiles: int, pairs: int):
    rem = tiles % pairs
    if tiles > pairs and rem > 0 and 2 * rem <= pairs:
        return tiles - rem, tiles + rem
    return tiles, tiles


@pytest.mark.parametrize("pairs", [1, 2, 37, 74])
def test_pair_units_cover_every_tile_once(pairs):
    """gemm_fp8.cu pair_units / pair_unit: units below full_units are whole tiles; the rest
    are (tile, half) with tile = full + (u - full) // 2. Every tile must be produced exactly
    once, whole or as both halves, and the split must only happen for a thin last wave."""
    for tiles in itertools.chain(range(1, 400), (1024, 1376, 4096)):
        full, units = _pair_units(tiles, pairs)
        got = {}
        for u in range(units):
            if u < full:
                got.setdefault(u, []).append("whole")
            else:
                got.setdefault(full + (u - full) // 2, []).append((u - full) & 1)
        assert sorted(got) == list(range(tiles))
        for t, parts in got.items():
            assert parts == ["whole"] or sorted(parts) == [0, 1]
        if units != tiles:
            waves_before = -(-tiles // pairs)
            assert units - full <= pairs and -(-full // pairs) + 1 == waves_before


def test_decode_warp_block_sequence_matches_its_consumption_order():
    """int4.cu: a warp requests blocks in the order (round, phase, tile) with a running source
    pointer; model the pointer and check it against the closed form
    ((r0 + t) * ngroups + p * warps + warp) * 1056 for several shapes."""
    blk, warps, round_tiles = 1056, 16, 5
    for (ngroups, t_begin, t_end, warp) in [(32, 0, 5, 3), (32, 4, 9, 15), (8, 0, 13, 7), (2, 10, 23, 1), (40, 7, 8, 9)]:
        my_phases = (ngroups - warp + warps - 1) // warps if warp < ngroups else 0
        tile_stride = ngroups * blk
        wmine = warp * blk
        r0, rt, p, t = t_begin, min(round_tiles, t_end - t_begin), 0, 0
        src = wmine + t_begin * tile_stride
        seq = []
        while my_phases > 0 and r0 < t_end:
            seq.append(src)
            src += tile_stride
            t += 1
            if t == rt:
                t = 0
                p += 1
                if p == my_phases:
                    p = 0
                    r0 += round_tiles
                    rt = min(round_tiles, t_end - r0)
                src = wmine + r0 * tile_stride + p * warps * blk
        want = [((rr + tt) * ngroups + pp * warps + warp) * blk
                for rr in range(t_begin, t_end, round_tiles)
                for pp in range(my_phases)
                for tt in range(min(round_tiles, t_end - rr))]
        assert seq == want


@pytest.mark.parametrize("share", [4, 5])
def test_decode_straight_line_order_is_the_general_order(share):
    """int4.cu, the one-round two-group path: block b is (group b // RT, tile b % RT) read from
    s0 or s1 + (b % RT) * tile_stride into ring slot b % depth. That must be the order of the
    general sequence (whose first `depth` requests the kernel's prologue has already issued),
    a block's slot must be free when it is requested (block b - depth has been read), and the
    activations copied with the first request after the wait must have landed at b = RT."""
    blk, warps, depth, ngroups = 1056, 16, 3, 32
    tile_stride = ngroups * blk
    for warp in (0, 7, 15):
        for t_begin in (0, 9, 683):
            s0 = warp * blk + t_begin * tile_stride
            s1 = s0 + warps * blk
            straight = [(s0 if b < share else s1) + (b % share) * tile_stride for b in range(2 * share)]
            general = [((t_begin + t) * ngroups + p * warps + warp) * blk for p in range(2) for t in range(share)]
            assert straight == general
    # ring discipline: before step b the committed groups are blocks 0 .. depth - 1 + b; waiting for
    # all but the newest depth - 1 leaves blocks 0 .. b complete; the x copies ride in group `depth`
    for b in range(2 * share):
        committed = depth + b
        complete = committed - (depth - 1)
        assert complete == b + 1
        if b + depth < 2 * share:
            assert (b + depth) % depth == b % depth  # the slot just read is the one refilled
    assert share >= depth  # group `depth` (first commit after the wait) is complete from step depth on


@pytest.mark.parametrize("tiles,sms", [(688, 148), (1376, 148), (86, 148), (149, 148), (1, 148), (4096, 132)])
def test_decode_tile_partition_covers_every_tile_once(tiles, sms):
    """int4.cu: the host passes share_q = tiles // grid and share_r = tiles % grid; CTA b owns
    [b * q + min(b, r), + q + (b < r)). The shares must tile [0, tiles) in order and differ by
    at most one; 688 tiles on 148 CTAs give only shares of 4 and 5 (the straight-line path)."""
    grid = min(tiles, sms)
    q, r = divmod(tiles, grid)
    end = 0
    shares = set()
    for b in range(grid):
        t_begin = b * q + min(b, r)
        t_end = t_begin + q + (1 if b < r else 0)
        assert t_begin == end and t_end > t_begin
        shares.add(t_end - t_begin)
        end = t_end
    assert end == tiles and max(shares) - min(shares) <= 1
    if (tiles, sms) == (688, 148):
        assert shares == {4, 5}


def _tile_coords(tile, m_tiles, n_tiles, group):
    """Integer model of the persistent GEMM scheduler's tile order (tile_coords in gemm_fp8.cu):
    grouped raster, odd groups walking the N tiles backwards."""
    per_group = n_tiles * group
    gid, off = divmod(tile, per_group)
    first_m = gid * group
    gsz = min(group, m_tiles - first_m)
    tm, tn = first_m + off % gsz, off // gsz
    if gid & 1:
        tn = n_tiles - 1 - tn
    return tm, tn


def test_gemm_tile_order_is_a_bijection_and_turns_around_between_groups():
    # the reference validates its swizzle on these grids (src/ptx_emitter.rs:7477-7513); the
    # byte-sized groups of this build range from 1 to all M tiles
    for m_tiles, n_tiles in [(1, 1), (1, 7), (7, 1), (8, 8), (32, 32), (16, 86), (33, 17), (5, 3), (100, 9)]:
        for group in (1, 2, 3, 8, 16, 32, 1000):
            group = min(group, m_tiles)
            seen = [_tile_coords(t, m_tiles, n_tiles, group) for t in range(m_tiles * n_tiles)]
            assert sorted(seen) == [(m, n) for m in range(m_tiles) for n in range(n_tiles)]
            if m_tiles > group:
                # the last N tile of the first group is the first N tile of the second
                last_of_first = seen[n_tiles * group - 1]
                first_of_second = seen[n_tiles * group]
                assert last_of_first[1] == first_of_second[1] == n_tiles - 1
