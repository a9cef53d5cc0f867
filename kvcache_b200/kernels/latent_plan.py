"""Work list of the attention kernel over shared key rows (csrc/latent_flash.cu).

All heads of a token read the same cached rows, so the kernel's rows are (token, head) pairs: a request that brings
`count` tokens has count * H rows, cut into tiles of BM rows; a tile sees the keys up to its last token's position.
Every tile is cut into the same number of splits over its keys - as many as bring the launch to about `blocks_wanted`
blocks, so that a few decoded tokens with long contexts still fill the GPU - and the splits of a tile are added up by
a second kernel in their order.  The number of splits follows from the number of tiles alone; steps of decoded tokens
with the same number of requests therefore have the same launches and can be replayed from one CUDA graph.
With a window a tile's keys start at the tile of 64 keys that holds the first key its first row sees; what lies before
is neither read nor expected in the cache (a windowed cache entry has given those pages back).
"""
from __future__ import annotations

import functools
from typing import Dict, Tuple

import numpy as np

from ..parts.base import StepPlanner

KEY_TILE = 64
SMALL_TILE, LARGE_TILE = 16, 64      # rows of a tile: 16 while every request's rows fit one such tile, else 64
MAX_SPLITS = 32


@functools.lru_cache(maxsize=1024)
def _plan(segments: tuple, heads: int, blocks_wanted: int, large_tile: int = LARGE_TILE, window: int = 0):
    """segments: (segment index, tokens cached, tokens brought).  Returns (int32 [items, 4]: segment, first row, first
    key, end of keys; tiles; splits per tile; rows of a tile)."""
    bm = SMALL_TILE if all(count * heads <= SMALL_TILE for _, _, count in segments) else large_tile
    tiles = []
    for seg, start, count in segments:
        for m0 in range(0, count * heads, bm):
            last_token = min(count - 1, (m0 + bm - 1) // heads)
            first_key = max(0, start + m0 // heads - window + 1) // KEY_TILE * KEY_TILE if window else 0
            tiles.append((seg, m0, start + last_token + 1, first_key))
    tiles.sort(key=lambda t: t[3] - t[2])        # the tiles with the most keys first
    nsplit = max(1, min(MAX_SPLITS, blocks_wanted // len(tiles)))
    items = []
    for seg, m0, kv_end, first_key in tiles:
        per = -(-(-(-(kv_end - first_key) // KEY_TILE)) // nsplit) * KEY_TILE          # keys of a split: whole key tiles
        for s in range(nsplit):
            kb = min(first_key + s * per, kv_end)
            items.append((seg, m0, kb, min(kv_end, kb + per)))
    array = np.asarray(items, dtype=np.int32).reshape(-1, 4)
    array.setflags(write=False)
    return array, len(tiles), nsplit, bm


class LatentAttentionPlanner(StepPlanner):
    def __init__(self, heads: int, blocks_wanted: int, large_tile: int = LARGE_TILE, window: int = 0):
        """`large_tile`: rows of a tile in steps that bring more than `SMALL_TILE` rows of a request (64, or 32 where the
        kernel's shared memory holds two key stages only beside the smaller tile).  `window`: keys a query sees, its own
        included (0: all)."""
        self.heads, self.blocks_wanted, self.large_tile, self.window = heads, blocks_wanted, large_tile, int(window or 0)
        self.name = self.plan_name(heads, blocks_wanted, large_tile, self.window)

    @staticmethod
    def plan_name(heads: int, blocks_wanted: int, large_tile: int = LARGE_TILE, window: int = 0) -> str:
        return f"latent_attention.h{heads}.b{blocks_wanted}.t{large_tile}" + (f".w{window}" if window else "")

    def sections(self, num_tokens: int, num_segments: int) -> Dict[str, int]:
        tiles = num_tokens * self.heads // self.large_tile + 2 * num_segments
        return {"items": 4 * max(tiles, self.blocks_wanted + num_segments)}

    def plan(self, starts, counts) -> Tuple[Dict[str, np.ndarray], Dict[str, int]]:
        segments = tuple((i, int(s), int(c)) for i, (s, c) in enumerate(zip(starts, counts)))
        items, tiles, nsplit, bm = _plan(segments, self.heads, self.blocks_wanted, self.large_tile, self.window)
        return {"items": items.reshape(-1)}, {"items": len(items), "tiles": tiles, "nsplit": nsplit, "bm": bm}
