"""Oracle for the radial tile masks (numpy, CPU).  Test infrastructure only.

Two mask builders:

* ``radial_log_mask`` restates the reference's ``gen_log_mask_shrinked`` +
  ``MaskMap.query_log_mask`` + the expansion in ``RadialSageAttentionImpl``
  (ksana/operations/attention/backends/radial_sage_attn/attn_mask.py:20-145 and
  radial_sage_attn.py:138-160) and is pinned against them by the golden fixtures.
* ``bernoulli_frame_mask`` is the mask the benchmark's configuration 5 specifies for the 720p
  shape, which the reference itself cannot build (its constructor requires the
  latent H and W to be multiples of block_size/8, radial_sage_attn.py:126-127):
  same-frame tiles always kept, a cross-frame tile kept with probability
  2^-|dframe| from a seeded generator.  A tile belongs to the frame of its
  first token.
"""

from __future__ import annotations

import numpy as np


def _window_width(dist, tpf, decay, bs):
    """attn_mask.py:53-62."""
    if dist < 1:
        return tpf
    if dist == 1:
        return tpf // 2
    return max(2 ** tpf.bit_length() / 2 ** dist.bit_length() * decay, bs)


def _frame_pair_kept(dist, tpf, bs):
    """attn_mask.py:35-50: beyond the point where the decayed length drops under a tile,
    only every (bs/len)-th frame distance survives."""
    length = 2 ** tpf.bit_length() / 2 ** dist.bit_length()
    if length >= bs:
        return True
    return dist % int(bs / length) == 0


def _shrink(mask, bs):
    """attn_mask.py:20-32: a tile survives when more than 60% of its non-empty columns
    are more than 1/3 dense."""
    nb = mask.shape[0] // bs
    nbc = mask.shape[1] // bs
    m = mask[: nb * bs, : nbc * bs].reshape(nb, bs, nbc, bs)
    dens = m.sum(axis=1).astype(np.float32) / np.float32(bs)  # [nb, nbc, bs]
    nonzero = (dens > 0).sum(axis=-1)
    high = (dens > np.float32(1 / 3)).sum(axis=-1)
    frac = high.astype(np.float32) / (nonzero.astype(np.float32) + np.float32(1e-9))
    return frac > np.float32(0.6)


def frame_pair_tiles(s, video_tokens, num_frame, bs=128, decay=0.5):
    """gen_log_mask_shrinked (attn_mask.py:65-112) -> bool [s//bs, s//bs]."""
    nb = s // bs
    out = np.zeros((nb, nb), dtype=bool)
    tpf = video_tokens // num_frame
    border = video_tokens // bs
    out[border:] = True
    out[:, border:] = True
    r = np.arange(tpf)
    absdiff = np.abs(r[None, :] - r[:, None])
    span = ((tpf - 1) // bs + 1) * bs
    for i in range(num_frame):
        for j in range(num_frame):
            if j == 0:
                local = np.ones((tpf, tpf), dtype=bool)  # attention sink column
            else:
                dist = abs(i - j)
                local = absdiff <= _window_width(dist, tpf, decay, bs)
                if not _frame_pair_kept(dist, tpf, bs):
                    local = np.zeros_like(local)
            rr, rc = (i * tpf) % bs, (j * tpf) % bs
            padded = np.zeros((rr + span, rc + span), dtype=bool)
            padded[rr : rr + tpf, rc : rc + tpf] = local
            blk = _shrink(padded, bs)
            r0, c0 = (i * tpf) // bs, (j * tpf) // bs
            r1, c1 = min(r0 + blk.shape[0], nb), min(c0 + blk.shape[1], nb)
            out[r0:r1, c0:c1] |= blk[: r1 - r0, : c1 - c0]
    return out


def radial_log_mask(seq_len, video_tokens, num_frame, bs=128, decay=0.5):
    """MaskMap.query_log_mask (attn_mask.py:123-137): ones outside the video border."""
    nb = seq_len // bs
    full = np.ones((nb, nb), dtype=bool)
    inner = frame_pair_tiles(seq_len, video_tokens, num_frame, bs, decay)
    b = video_tokens // bs
    full[:b, :b] = inner[:b, :b]
    return full


def expand_to_q128_k64(tile_mask, bs):
    """radial_sage_attn.py:155-160: bs 128 -> repeat columns x2; bs 64 -> max over row pairs."""
    if bs == 128:
        return np.repeat(tile_mask, 2, axis=1)
    assert bs == 64
    return tile_mask.reshape(tile_mask.shape[0] // 2, 2, tile_mask.shape[1]).max(axis=1)


def bernoulli_frame_mask(L, tokens_per_frame, seed=0, tile=128):
    """The benchmark's configuration-5 mask -> bool [ceil(L/128), ceil(L/128)] (128 x 128 tiles)."""
    nt = (L + tile - 1) // tile
    frame = (np.arange(nt) * tile) // tokens_per_frame
    d = np.abs(frame[:, None] - frame[None, :])
    rng = np.random.RandomState(seed)
    u = rng.random_sample((nt, nt))
    return (d == 0) | (u < np.exp2(-d.astype(np.float64)))


def tile_lists(mask_q128_k64):
    """Compact per-Q-block lists of KV tiles for the block-sparse kernel.

    mask [nq, nk64] bool -> (offsets int32 [nq+1], entries int32 [nnz]); an entry is
    kv_tile * 4 + halves, kv_tile indexing 128-token tiles, halves bit0/bit1 marking which
    64-token half of the tile is kept.
    """
    m = np.asarray(mask_q128_k64).astype(bool)
    nq, nk = m.shape
    if nk % 2:
        m = np.concatenate([m, np.zeros((nq, 1), dtype=bool)], axis=1)
        nk += 1
    halves = m[:, 0::2].astype(np.int32) + 2 * m[:, 1::2].astype(np.int32)
    offs = [0]
    ents = []
    for r in range(nq):
        idx = np.nonzero(halves[r])[0]
        ents.append(idx.astype(np.int32) * 4 + halves[r, idx])
        offs.append(offs[-1] + len(idx))
    ent = np.concatenate(ents) if ents else np.zeros(0, np.int32)
    return np.asarray(offs, np.int32), ent.astype(np.int32)
