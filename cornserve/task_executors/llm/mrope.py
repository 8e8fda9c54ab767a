"""M-RoPE position ids for prompts with image / video placeholders (Qwen2-VL family).

Text tokens advance all three rows together; the tokens of one image get (t, h, w) grid coordinates
offset by the running position; text after an image resumes at ``max(position) + 1``.
"""

from __future__ import annotations

import numpy as np


def mrope_positions(
    token_ids: np.ndarray,
    grids_thw: list[tuple[int, int, int]],
    image_token_id: int,
    video_token_id: int = -1,
    merge: int = 2,
    second_per_grid: list[float] | None = None,
    tokens_per_second: float = 2.0,
) -> tuple[np.ndarray, int]:
    """Returns ``(positions [3, T] int32, next_position)`` where ``next_position`` is the position
    id of the first generated token."""
    T = int(token_ids.shape[0])
    pos = np.zeros((3, T), dtype=np.int32)
    is_mm = (token_ids == image_token_id) | (token_ids == video_token_id)
    i, cur, g = 0, 0, 0
    while i < T:
        if not is_mm[i]:
            j = i
            while j < T and not is_mm[j]:
                j += 1
            n = j - i
            pos[:, i:j] = cur + np.arange(n, dtype=np.int32)[None, :]
            cur += n
            i = j
            continue
        if g >= len(grids_thw):
            raise ValueError("more placeholder runs than grids")
        t, h, w = grids_thw[g]
        gh, gw = h // merge, w // merge
        n = t * gh * gw
        if i + n > T or not is_mm[i: i + n].all():
            raise ValueError(f"placeholder run {g} does not match its grid {grids_thw[g]}")
        tt = np.repeat(np.arange(t), gh * gw)
        if token_ids[i] == video_token_id and second_per_grid is not None:
            tt = (tt * second_per_grid[g] * tokens_per_second).astype(np.int64)
        hh = np.tile(np.repeat(np.arange(gh), gw), t)
        ww = np.tile(np.arange(gw), t * gh)
        pos[0, i: i + n] = cur + tt
        pos[1, i: i + n] = cur + hh
        pos[2, i: i + n] = cur + ww
        cur = int(pos[:, i: i + n].max()) + 1
        i += n
        g += 1
    return pos, cur
