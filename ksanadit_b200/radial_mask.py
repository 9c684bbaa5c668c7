"""Radial tile masks for the block-sparse attention backend (host-side set-up, cached by the caller).

Same mask semantics as KsanaDiT's ``MaskMap`` / ``gen_log_mask_shrinked`` / ``shrink_mask_strict``
(ksana/operations/attention/backends/radial_sage_attn/attn_mask.py:20-145) and the expansion to the
kernel's (128 x 64) granularity (radial_sage_attn.py:155-160).  The frame-pair pattern depends only on
|i - j| (and on j == 0, the attention-sink column), so each distinct pattern is built and shrunk to
tiles once per (distance, row offset, column offset) instead of once per frame pair.
"""

from __future__ import annotations

import numpy as np


def _pair_pattern(dist: int, tpf: int, bs: int, decay: float, sink: bool) -> np.ndarray:
    """Token-level mask [tpf, tpf] of one frame pair."""
    if sink:
        return np.ones((tpf, tpf), dtype=bool)
    if dist == 0:
        width = tpf
    elif dist == 1:
        width = tpf // 2
    else:
        width = max(2 ** tpf.bit_length() / 2 ** dist.bit_length() * decay, bs)
    length = 2 ** tpf.bit_length() / 2 ** dist.bit_length()
    if length < bs and dist % int(bs / length) != 0:
        return np.zeros((tpf, tpf), dtype=bool)
    idx = np.arange(tpf)
    return np.abs(idx[None, :] - idx[:, None]) <= width


def _to_tiles(pattern: np.ndarray, row_off: int, col_off: int, bs: int) -> np.ndarray:
    """Places the pattern at (row_off, col_off) inside a tile grid and keeps a tile when more than 60% of its
    non-empty columns are more than one third dense."""
    tpf = pattern.shape[0]
    span = ((tpf - 1) // bs + 1) * bs
    # the reference pads the pair to (offset + span) and shrinks whole tiles only (attn_mask.py:20-32,98-105): what
    # spills past the last whole tile of the padded block is dropped, also when the frame does not end on a tile edge
    rows, cols = (row_off + span) // bs, (col_off + span) // bs
    canvas = np.zeros((row_off + span, col_off + span), dtype=bool)
    canvas[row_off:row_off + tpf, col_off:col_off + tpf] = pattern
    canvas = canvas[:rows * bs, :cols * bs]
    dens = canvas.reshape(rows, bs, cols, bs).sum(axis=1, dtype=np.int64).astype(np.float32) / np.float32(bs)
    nonzero = (dens > 0).sum(axis=-1).astype(np.float32)
    high = (dens > np.float32(1 / 3)).sum(axis=-1).astype(np.float32)
    return high / (nonzero + np.float32(1e-9)) > np.float32(0.6)


def build_radial_tile_mask(seq_len: int, video_tokens: int, num_frame: int, block_size: int = 128, decay_factor: float = 0.5):
    """bool [seq_len // bs, seq_len // bs]: True = keep the tile.  Rows/columns past the video are kept."""
    bs = block_size
    nb = seq_len // bs
    tpf = video_tokens // num_frame
    border = video_tokens // bs
    inner = np.zeros((nb, nb), dtype=bool)
    cache: dict = {}
    for i in range(num_frame):
        ro = (i * tpf) % bs
        r0 = (i * tpf) // bs
        for j in range(num_frame):
            co = (j * tpf) % bs
            key = (0 if j == 0 else abs(i - j), j == 0, ro, co)
            blk = cache.get(key)
            if blk is None:
                blk = _to_tiles(_pair_pattern(abs(i - j), tpf, bs, decay_factor, j == 0), ro, co, bs)
                cache[key] = blk
            c0 = (j * tpf) // bs
            r1, c1 = min(r0 + blk.shape[0], nb), min(c0 + blk.shape[1], nb)
            inner[r0:r1, c0:c1] |= blk[: r1 - r0, : c1 - c0]
    out = np.ones((nb, nb), dtype=bool)
    out[:border, :border] = inner[:border, :border]
    return out


def expand_to_kernel_granularity(tile_mask: np.ndarray, block_size: int) -> np.ndarray:
    """[L/bs, L/bs] -> [L/128, L/64] (radial_sage_attn.py:155-160)."""
    if block_size == 128:
        return np.repeat(tile_mask, 2, axis=1)
    if block_size == 64:
        return tile_mask.reshape(tile_mask.shape[0] // 2, 2, tile_mask.shape[1]).max(axis=1)
    raise ValueError(f"block_size must be 64 or 128, got {block_size}")


def bernoulli_frame_tile_mask(L: int, tokens_per_frame: int, seed: int = 0, tile: int = 128) -> np.ndarray:
    """128 x 128 tile mask: same-frame tiles kept, cross-frame tiles kept with probability 2^-|dframe|
    (a tile belongs to the frame of its first token).  Used for shapes the radial rule cannot tile."""
    nt = (L + tile - 1) // tile
    frame = (np.arange(nt) * tile) // tokens_per_frame
    d = np.abs(frame[:, None] - frame[None, :])
    u = np.random.RandomState(seed).random_sample((nt, nt))
    return (d == 0) | (u < np.exp2(-d.astype(np.float64)))


def compact_tile_lists(mask_q128_k64: np.ndarray):
    """Mask [nq, nk64] -> (offsets int32 [nq+1], entries int32 [nnz]) in the kernel's list format:
    entry = kv_tile * 4 + keep bits (bit 0: first 64 tokens of the 128-token tile, bit 1: last 64)."""
    m = np.asarray(mask_q128_k64, dtype=bool)
    if m.shape[1] % 2:
        m = np.concatenate([m, np.zeros((m.shape[0], 1), dtype=bool)], axis=1)
    halves = m[:, 0::2].astype(np.int32) | (m[:, 1::2].astype(np.int32) << 1)
    rows, cols = np.nonzero(halves)
    counts = np.bincount(rows, minlength=m.shape[0])
    offsets = np.zeros(m.shape[0] + 1, dtype=np.int32)
    np.cumsum(counts, out=offsets[1:])
    entries = (cols.astype(np.int32) * 4 + halves[rows, cols]).astype(np.int32)
    return offsets, entries


def longest_first_order(offsets: np.ndarray) -> np.ndarray:
    """Permutation of the Q blocks by decreasing list length (stable), for the kernel's ``q_order`` argument."""
    counts = np.diff(np.asarray(offsets, dtype=np.int64))
    return np.argsort(-counts, kind="stable").astype(np.int32)


def pair_tile_lists(offsets: np.ndarray, entries: np.ndarray):
    """Per-block lists (``compact_tile_lists``) -> per-pair lists for the kernel that keeps Q blocks 2i and 2i+1 in
    one CTA: (pair_offsets int32 [ceil(nq/2)+1], pair_entries int32 [nnz]), the union of the two blocks' KV tiles in
    ascending order, entry = kv_tile * 16 + keep bits of block 2i + (keep bits of block 2i+1 << 2)."""
    offsets = np.asarray(offsets, dtype=np.int64)
    entries = np.asarray(entries, dtype=np.int64)
    nq = offsets.size - 1
    npairs = (nq + 1) // 2
    if entries.size == 0:
        return np.zeros(npairs + 1, dtype=np.int32), np.zeros(0, dtype=np.int32)
    block = np.repeat(np.arange(nq, dtype=np.int64), np.diff(offsets))  # Q block of every entry
    tile, keep = entries >> 2, entries & 3
    ntiles = int(tile.max()) + 1
    key = (block >> 1) * ntiles + tile                      # (pair, kv tile)
    bits = keep << (2 * (block & 1))
    uniq, inv = np.unique(key, return_inverse=True)          # sorted: by pair, then by tile
    merged = np.zeros(uniq.size, dtype=np.int64)
    np.bitwise_or.at(merged, inv, bits)
    pair = uniq // ntiles
    counts = np.bincount(pair, minlength=npairs)
    pair_offsets = np.zeros(npairs + 1, dtype=np.int32)
    np.cumsum(counts, out=pair_offsets[1:])
    pair_entries = ((uniq % ntiles) * 16 + merged).astype(np.int32)
    return pair_offsets, pair_entries
