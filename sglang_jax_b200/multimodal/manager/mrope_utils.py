"""3-D rotary positions for vision-language prompts (reference
`python/sgl_jax/srt/multimodal/manager/mrope_utils.py`).

Text tokens advance the three streams (temporal, height, width) together.  The tokens of an image
or video keep the running position in the temporal stream (videos add `frame * interval`) and
count rows / columns of the merged patch grid in the other two; the text that follows resumes at
`start + max(grid_h, grid_w)`.  `delta` is what must be added to a generated token's index to get
its position."""

from __future__ import annotations

import numpy as np


def get_rope_index(input_ids, image_grid_thw=None, video_grid_thw=None, *, image_token_id: int,
                   video_token_id: int | None = None, spatial_merge_size: int = 2, tokens_per_second: float = 1.0,
                   second_per_grid_ts=None) -> tuple[np.ndarray, int]:
    """`input_ids [T]` with one placeholder token per merged patch -> (`positions i32 [3, T]`, `delta`)."""
    ids = np.asarray(input_ids)
    T = len(ids)
    images = [tuple(int(v) for v in g) for g in (np.asarray(image_grid_thw).reshape(-1, 3) if image_grid_thw is not None else [])]
    videos = [tuple(int(v) for v in g) for g in (np.asarray(video_grid_thw).reshape(-1, 3) if video_grid_thw is not None else [])]
    secs = list(second_per_grid_ts) if second_per_grid_ts is not None else [1.0] * len(videos)
    out = np.zeros((3, T), np.int32)
    cur, i, ii, vi = 0, 0, 0, 0
    m = spatial_merge_size
    while i < T:
        tok = ids[i]
        is_img = tok == image_token_id
        is_vid = video_token_id is not None and tok == video_token_id
        if not (is_img or is_vid):
            out[:, i] = cur
            cur += 1
            i += 1
            continue
        if is_img:
            if ii >= len(images):
                raise ValueError("more image placeholder runs than image grids")
            t, h, w = images[ii]
            ii += 1
            interval = 0.0
        else:
            if vi >= len(videos):
                raise ValueError("more video placeholder runs than video grids")
            t, h, w = videos[vi]
            interval = float(tokens_per_second) * float(secs[vi])
            vi += 1
        gh, gw = h // m, w // m
        n = t * gh * gw
        if i + n > T or not np.all(ids[i:i + n] == tok):
            raise ValueError(f"placeholder run at {i} is shorter than its {t}x{gh}x{gw} grid")
        f = np.arange(n) // (gh * gw)
        out[0, i:i + n] = cur + (f * interval).astype(np.int32)
        out[1, i:i + n] = cur + (np.arange(n) % (gh * gw)) // gw
        out[2, i:i + n] = cur + np.arange(n) % gw
        cur = int(out[:, i:i + n].max()) + 1 if n else cur
        cur = max(cur, int(out[0, i]) + max(gh, gw)) if n else cur
        i += n
    delta = (int(out.max()) + 1 - T) if T else 0
    return out, delta
