"""CPU restatement of the rulebook plan of the output-stationary MVMR kernel (TEST INFRASTRUCTURE).

The plan has no counterpart in the reference (the closest is the bucket table of its fused
gather-sum engine, sparse_engines/fused_point_conv.py:785-870); this numpy version states what
``pcx_mvmr_plan_build`` must produce, so that the device builder can be checked bit for bit:

  signature   bit (tap mod 32) for every tap that touches an output row
  perm        output rows in ascending signature order (stable), for a cubic kernel of at most 32 taps
              in ascending (kernel planes used, signature) order; padded with -1 to blocks of 128
  key         ((block * K + tap) * 128 + slot) of every triplet, block / slot = position in perm
  entries     triplets in ascending key order (stable): (slot, position within equal keys, row)
  tile_offs   exclusive sum of the triplet counts per (block, tap)
"""
import numpy as np

ROWS = 128


def build(scatter, gather, tap, n_out, K):
    scatter = np.asarray(scatter, np.int64)
    gather = np.asarray(gather, np.int64)
    tap = np.asarray(tap, np.int64)
    sig = np.zeros(n_out, np.int64)
    np.bitwise_or.at(sig, scatter, 1 << (tap & 31))
    order = np.argsort(sig, kind="stable")
    ks = round(K ** (1 / 3))
    if ks ** 3 == K and 1 < K <= 32:
        # cubic kernel: rows first by the kx / ky / kz planes of the kernel they use (kz most
        # significant), then by signature; stable in both
        taps = np.arange(K)
        planes = np.zeros(n_out, np.int64)
        for axis, coord in enumerate((taps // (ks * ks), (taps // ks) % ks, taps % ks)):
            for v in range(ks):
                uses = (sig & int(np.sum(1 << taps[coord == v]))) != 0
                planes |= uses.astype(np.int64) << (axis * ks + v)
        order = np.lexsort((sig, planes))
    nblocks = (n_out + ROWS - 1) // ROWS
    perm = np.full(nblocks * ROWS, -1, np.int64)
    perm[:n_out] = order
    rank = np.empty(n_out, np.int64)
    rank[order] = np.arange(n_out)
    r = rank[scatter]
    key = (((r >> 7) * K + tap) << 7) | (r & 127)
    by_key = np.argsort(key, kind="stable")
    key_sorted, rows = key[by_key], gather[by_key]
    counts = np.bincount(key_sorted >> 7, minlength=nblocks * K)
    tile_offs = np.concatenate(([0], np.cumsum(counts)))
    same = np.concatenate(([False], key_sorted[1:] == key_sorted[:-1]))
    pos = np.zeros(len(key_sorted), np.int64)
    run = 0
    for t in range(len(key_sorted)):
        run = run + 1 if same[t] else 0
        pos[t] = run
    return dict(perm=perm, tile_offs=tile_offs, key=key_sorted, slot=key_sorted & 127, pos=pos, rows=rows,
                nblocks=nblocks)
