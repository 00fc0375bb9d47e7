"""Media processor: images / videos -> bf16 patch rows, expanded placeholders and three-axis positions.

Steps (docs/maintainer/qwen3.6-27b-model.md section 9, src/targets/qwen3_6/impl/frontend/processor.cpp:75-125,
495-520): decode, choose dimensions aligned to the 32-pixel merge factor within a pixel budget, bicubic
resize, normalise to [-1, 1], pack channel-major 2 x 16 x 16 temporal-spatial patches into bf16 rows of
width 1536 (images repeat their frame to fill the temporal pair), expand each chat placeholder to one pad
token per merged 2 x 2 patch block, and build [T, 3] (temporal, height, width) positions plus the
`rope_delta` that turns later scalar decode indices into rope positions.

Decoding uses Pillow (still images and multi-frame files); callers can also pass frames as uint8 arrays.
There is no container demuxer here: a video is a sequence of frames with a frame rate.
"""
from __future__ import annotations

import base64
import io
import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

PATCH, TEMPORAL, MERGE = 16, 2, 2
FACTOR = PATCH * MERGE
PATCH_FEATURES = 3 * TEMPORAL * PATCH * PATCH
IMAGE_PAD, VIDEO_PAD = "<|image_pad|>", "<|video_pad|>"
VISION_START, VISION_END = "<|vision_start|>", "<|vision_end|>"
IMAGE_TOKEN_ID, VIDEO_TOKEN_ID = 248056, 248057   # processor.cpp:45-46
MAX_RAW_PATCHES, MAX_VISION_TOKENS = 131072, 32768


@dataclass
class MediaOptions:
    image_min_pixels: int = 64 * 1024
    image_max_pixels: int = 16 * 1024 * 1024
    video_min_pixels: int = 128 * 1024
    video_max_pixels: int = 24 * 1024 * 1024   # frames x height x width
    video_fps: float = 2.0
    video_min_frames: int = 4
    video_max_frames: int = 768
    max_source_bytes: int = 256 * 1024 * 1024


@dataclass
class MediaItem:
    modality: str                      # "image" | "video"
    grid: Tuple[int, int, int]         # (temporal groups, height, width) in patches
    patches: torch.Tensor              # bf16 [t * h * w, 1536], merge-block order inside each temporal group
    timestamps: List[float] = field(default_factory=list)   # one per temporal group (video)

    @property
    def frame_tokens(self) -> int:
        return (self.grid[1] // MERGE) * (self.grid[2] // MERGE)

    @property
    def n_tokens(self) -> int:
        return self.grid[0] * self.frame_tokens


@dataclass
class PreparedPrompt:
    """A tokenised prompt with media: everything the runtime needs for a multimodal prefill."""
    ids: List[int]
    positions: np.ndarray        # int32 [T, 3] temporal / height / width
    rope_delta: int              # next position - token count
    items: List[MediaItem]
    embed_rows: np.ndarray       # int32 [V] token index of every pad token, in item / frame / block order

    @property
    def grids(self) -> List[Tuple[int, int, int]]:
        return [it.grid for it in self.items]

    def patches(self) -> torch.Tensor:
        return torch.cat([it.patches for it in self.items]) if self.items else torch.zeros((0, PATCH_FEATURES), dtype=torch.bfloat16)


# ---------------------------------------------------------------------------------------- geometry
def _round_even(v: float) -> int:
    return int(np.rint(v))   # ties to even, like nearbyint


def smart_resize_image(height: int, width: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    if height <= 0 or width <= 0 or min_pixels <= 0 or max_pixels < min_pixels:
        raise ValueError("invalid image dimensions or pixel budget")
    if max(height, width) / min(height, width) > 200:
        raise ValueError("image aspect ratio exceeds 200")
    h = max(FACTOR, _round_even(height / FACTOR) * FACTOR)
    w = max(FACTOR, _round_even(width / FACTOR) * FACTOR)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(FACTOR, math.floor(height / beta / FACTOR) * FACTOR)
        w = max(FACTOR, math.floor(width / beta / FACTOR) * FACTOR)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / FACTOR) * FACTOR
        w = math.ceil(width * beta / FACTOR) * FACTOR
    return h, w


def smart_resize_video(frames: int, height: int, width: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    if frames <= 0 or height < FACTOR or width < FACTOR or min_pixels <= 0 or max_pixels < min_pixels:
        raise ValueError("invalid video dimensions or pixel budget")
    h = _round_even(height / FACTOR) * FACTOR
    w = _round_even(width / FACTOR) * FACTOR
    volume = frames * h * w
    if volume > max_pixels:
        beta = math.sqrt(frames * height * width / max_pixels)
        h = max(FACTOR, math.floor(height / beta / FACTOR) * FACTOR)
        w = max(FACTOR, math.floor(width / beta / FACTOR) * FACTOR)
    elif volume < min_pixels:
        beta = math.sqrt(min_pixels / (frames * height * width))
        h = math.ceil(height * beta / FACTOR) * FACTOR
        w = math.ceil(width * beta / FACTOR) * FACTOR
    return h, w


def sample_video_frames(n_frames: int, source_fps: float, target_fps: float, min_frames: int, max_frames: int) -> List[int]:
    """Indices of the frames kept: about `target_fps` per second, an even count within [min, max]."""
    if n_frames <= 0 or source_fps <= 0:
        raise ValueError("video has no frames")
    want = n_frames / source_fps * target_fps
    want = int(min(max(want, min_frames), max_frames, n_frames))
    want = max(TEMPORAL, want - want % TEMPORAL)
    return [int(v) for v in np.rint(np.linspace(0, n_frames - 1, want))]


def video_timestamps(indices: Sequence[int], fps: float) -> List[float]:
    """Mean time of each temporal pair (processor.cpp:332-345); an odd tail repeats its last frame."""
    idx = list(indices)
    if len(idx) % TEMPORAL:
        idx.append(idx[-1])
    return [(idx[2 * t] + idx[2 * t + 1]) / (2.0 * fps) for t in range(len(idx) // 2)]


# ---------------------------------------------------------------------------------------- pixels
def decode_media(source) -> np.ndarray:
    """uint8 [F, H, W, 3] from a path, bytes, a data: URI, a Pillow image or an array ([H, W, 3] or [F, H, W, 3])."""
    if isinstance(source, np.ndarray):
        arr = source
        if arr.ndim == 3:
            arr = arr[None]
        if arr.ndim != 4 or arr.shape[-1] != 3 or arr.dtype != np.uint8:
            raise ValueError("frames must be uint8 [F, H, W, 3]")
        return arr
    from PIL import Image, ImageSequence
    if isinstance(source, str) and source.startswith("data:"):
        head, _, payload = source.partition(",")
        source = base64.b64decode(payload) if head.endswith(";base64") else payload.encode()
    if isinstance(source, (bytes, bytearray)):
        source = io.BytesIO(bytes(source))
    img = source if isinstance(source, Image.Image) else Image.open(source)
    frames = [np.asarray(f.convert("RGB"), dtype=np.uint8) for f in ImageSequence.Iterator(img)]
    return np.stack(frames)


def _resize(frames: np.ndarray, h: int, w: int) -> np.ndarray:
    """Bicubic (a = -0.5, antialiased) resize of uint8 frames, result rounded back to uint8."""
    if frames.shape[1] == h and frames.shape[2] == w:
        return frames
    from PIL import Image
    return np.stack([np.asarray(Image.fromarray(f).resize((w, h), Image.BICUBIC), dtype=np.uint8) for f in frames])


def pack_patches(frames: np.ndarray) -> torch.Tensor:
    """uint8 [F, H, W, 3] (F even, H and W multiples of 32) -> bf16 [F/2 * H/16 * W/16, 1536].

    Row order: temporal pair, merge block row, merge block column, row inside the block, column inside the block;
    feature order: channel, frame of the pair, pixel row, pixel column.  Values are (v / 255 - 0.5) / 0.5 rounded
    to bf16 (nearest even)."""
    F, H, W, _ = frames.shape
    if F % TEMPORAL or H % FACTOR or W % FACTOR:
        raise ValueError("frames must come in temporal pairs with sides aligned to 32")
    x = torch.from_numpy(np.ascontiguousarray(frames)).float().div_(127.5).sub_(1.0)
    gh, gw = H // PATCH, W // PATCH
    # [T, t, by, iy, py, bx, ix, px, c] -> [T, by, bx, iy, ix, c, t, py, px]
    x = x.view(F // TEMPORAL, TEMPORAL, gh // MERGE, MERGE, PATCH, gw // MERGE, MERGE, PATCH, 3)
    x = x.permute(0, 2, 5, 3, 6, 8, 1, 4, 7).contiguous()
    return x.view(-1, PATCH_FEATURES).to(torch.bfloat16)


class MediaProcessor:
    def __init__(self, options: Optional[MediaOptions] = None):
        self.opt = options or MediaOptions()

    def image(self, source) -> MediaItem:
        frames = decode_media(source)[:1]
        h, w = smart_resize_image(frames.shape[1], frames.shape[2], self.opt.image_min_pixels, self.opt.image_max_pixels)
        frames = _resize(frames, h, w)
        pair = np.concatenate([frames, frames])   # a still image fills both frames of the temporal pair
        item = MediaItem("image", (1, h // PATCH, w // PATCH), pack_patches(pair))
        self._admit(item)
        return item

    def video(self, source, fps: float = 24.0) -> MediaItem:
        frames = decode_media(source)
        idx = sample_video_frames(frames.shape[0], fps, self.opt.video_fps, self.opt.video_min_frames,
                                  self.opt.video_max_frames)
        if len(idx) % TEMPORAL:
            idx.append(idx[-1])
        h, w = smart_resize_video(len(idx), frames.shape[1], frames.shape[2], self.opt.video_min_pixels,
                                  self.opt.video_max_pixels)
        picked = _resize(frames[idx], h, w)
        item = MediaItem("video", (len(idx) // TEMPORAL, h // PATCH, w // PATCH), pack_patches(picked),
                         video_timestamps(idx, fps))
        self._admit(item)
        return item

    @staticmethod
    def _admit(item: MediaItem) -> None:
        if item.patches.shape[0] > MAX_RAW_PATCHES or item.n_tokens > MAX_VISION_TOKENS:
            raise ValueError("media item exceeds the patch / vision-token limit")


# ---------------------------------------------------------------------------------------- prompt
def expand_placeholders(text: str, items: Sequence[MediaItem]) -> str:
    """Replaces the i-th media placeholder of a rendered chat by one pad token per merged block of item i.
    A video becomes one `<t seconds>` + vision-start / pads / vision-end run per temporal group."""
    out, cursor = [], 0
    for it in items:
        pad = IMAGE_PAD if it.modality == "image" else VIDEO_PAD
        whole = VISION_START + pad + VISION_END
        at = text.find(whole, cursor)
        if at < 0:
            raise ValueError("chat media count does not match the rendered placeholders")
        out.append(text[cursor:at])
        if it.modality == "image":
            out.append(VISION_START + pad * it.frame_tokens + VISION_END)
        else:
            for ts in it.timestamps:
                out.append(f"<{ts:.1f} seconds>" + VISION_START + pad * it.frame_tokens + VISION_END)
        cursor = at + len(whole)
    rest = text[cursor:]
    if (VISION_START + IMAGE_PAD + VISION_END) in rest or (VISION_START + VIDEO_PAD + VISION_END) in rest:
        raise ValueError("chat media count does not match the rendered placeholders")
    out.append(rest)
    return "".join(out)


def build_positions(ids: Sequence[int], items: Sequence[MediaItem], image_token: int = IMAGE_TOKEN_ID,
                    video_token: int = VIDEO_TOKEN_ID) -> Tuple[np.ndarray, int, np.ndarray]:
    """[T, 3] positions, rope_delta and the pad-token rows.  Text advances all three axes together; a run of pad
    tokens (one image, or one temporal group of a video) keeps the temporal axis at the run's start and walks
    the merged grid on the other two; the text after it resumes past the largest position used."""
    T = len(ids)
    pos = np.zeros((T, 3), dtype=np.int32)
    rows: List[int] = []
    runs = []   # (token id, merged h, merged w)
    for it in items:
        tok = image_token if it.modality == "image" else video_token
        runs.extend([(tok, it.grid[1] // MERGE, it.grid[2] // MERGE)] * it.grid[0])
    nxt, i, r = 0, 0, 0
    while i < T:
        if ids[i] in (image_token, video_token):
            if r >= len(runs) or runs[r][0] != ids[i]:
                raise ValueError("pad tokens do not match the media items")
            _, mh, mw = runs[r]
            n = mh * mw
            if i + n > T or any(ids[j] != ids[i] for j in range(i, i + n)):
                raise ValueError("a pad-token run is shorter than its media grid")
            yy, xx = np.divmod(np.arange(n, dtype=np.int32), mw)
            pos[i:i + n, 0] = nxt
            pos[i:i + n, 1] = nxt + yy
            pos[i:i + n, 2] = nxt + xx
            rows.extend(range(i, i + n))
            nxt += max(mh, mw)
            i += n
            r += 1
        else:
            pos[i] = nxt
            nxt += 1
            i += 1
    if r != len(runs):
        raise ValueError("fewer pad-token runs than media items")
    return pos, nxt - T, np.array(rows, dtype=np.int32)


def prepare_prompt(tokenizer, rendered_text: str, items: Sequence[MediaItem]) -> PreparedPrompt:
    """Expands the placeholders of a rendered chat, tokenises it and builds positions."""
    text = expand_placeholders(rendered_text, items)
    ids = list(tokenizer.encode(text))
    lookup = getattr(tokenizer, "token_id", None)
    img = lookup(IMAGE_PAD) if lookup else None
    vid = lookup(VIDEO_PAD) if lookup else None
    img = IMAGE_TOKEN_ID if img is None else img
    vid = VIDEO_TOKEN_ID if vid is None else vid
    pos, delta, rows = build_positions(ids, items, img, vid)
    return PreparedPrompt(ids, pos, delta, list(items), rows)


# ---------------------------------------------------------------------------------------- chat messages
def collect_media(messages: Sequence[dict]) -> List[Tuple[str, object]]:
    """(modality, source) of every image / video part of OpenAI-style messages, in rendering order (the system
    message first when it leads, as the chat template renders it)."""
    out: List[Tuple[str, object]] = []
    for m in messages:
        content = m.get("content")
        if not isinstance(content, (list, tuple)):
            continue
        for part in content:
            if not isinstance(part, dict):
                continue
            kind = part.get("type")
            if kind in ("image_url", "image", "input_image"):
                src = part.get("image_url", part.get("image"))
                out.append(("image", src.get("url") if isinstance(src, dict) else src))
            elif kind in ("video_url", "video"):
                src = part.get("video_url", part.get("video"))
                out.append(("video", src.get("url") if isinstance(src, dict) else src))
    return out


REMOTE_FETCH = {"enabled": False, "timeout_s": 10.0, "max_redirects": 3}   # set by the gateway (--allow-remote-media)


def fetch_remote(url: str, max_bytes: int, timeout_s: float = 10.0, max_redirects: int = 3) -> bytes:
    """Size-bounded HTTP(S) download of one media item: refuses other schemes, follows at most `max_redirects`
    redirects, refuses a declared or actual body larger than `max_bytes` (it stops reading at the limit), and turns
    every transport failure into a ValueError so that a bad URL fails the request, not the server.
    Reference: src/product/media_acquire/acquire.cpp (path / data: URI / HTTP(S), size-bounded)."""
    import urllib.error
    import urllib.request

    class Bounded(urllib.request.HTTPRedirectHandler):
        max_redirections = max_redirects
    if not url.startswith(("http://", "https://")):
        raise ValueError("only http:// and https:// media URLs are fetched")
    opener = urllib.request.build_opener(Bounded)
    try:
        with opener.open(urllib.request.Request(url, headers={"User-Agent": "ninfer-media/1"}), timeout=timeout_s) as r:
            if not r.geturl().startswith(("http://", "https://")):
                raise ValueError("media URL redirected to another scheme")
            declared = r.headers.get("Content-Length")
            if declared is not None and declared.isdigit() and int(declared) > max_bytes:
                raise ValueError("media source exceeds the byte limit")
            body = r.read(max_bytes + 1)
    except (urllib.error.URLError, OSError) as e:
        raise ValueError(f"media URL could not be fetched: {getattr(e, 'reason', e)}") from None
    if len(body) > max_bytes:
        raise ValueError("media source exceeds the byte limit")
    if not body:
        raise ValueError("media URL returned no content")
    return body


def acquire_source(source, allow_files: bool = False, max_bytes: int = 256 * 1024 * 1024):
    """Turns a message's media reference into something `decode_media` accepts.  `data:` URIs and in-memory
    objects always pass; `file://` / plain paths only when the gateway allows local files; remote URLs are fetched
    (size-bounded) only when the gateway switched remote media on."""
    if source is None:
        raise ValueError("media part has no source")
    if not isinstance(source, str):
        return source
    if source.startswith("data:"):
        if len(source) > max_bytes * 4 // 3 + 64:
            raise ValueError("media source exceeds the byte limit")
        return source
    if source.startswith(("http://", "https://")):
        if not REMOTE_FETCH["enabled"]:
            raise ValueError("remote media URLs are not fetched by this server; send a data: URI")
        return fetch_remote(source, max_bytes, REMOTE_FETCH["timeout_s"], REMOTE_FETCH["max_redirects"])
    path = source[len("file://"):] if source.startswith("file://") else source
    if not allow_files:
        raise ValueError("local media files are disabled on this gateway")
    import os
    if os.path.getsize(path) > max_bytes:
        raise ValueError("media source exceeds the byte limit")
    return path


def prepare_messages(tokenizer, rendered_text: str, messages: Sequence[dict], processor: "MediaProcessor",
                     allow_files: bool = False, video_fps: float = 24.0, pool=None,
                     checkpoint=None) -> Optional[PreparedPrompt]:
    """PreparedPrompt for chat messages with media parts, or None when there are none.  With a
    runtime.worker_pool.HostWorkerPool the items are decoded and resized on its threads (bounded queue;
    `checkpoint` lets a cancelled request stop waiting for a slot)."""
    refs = collect_media(messages)
    if not refs:
        return None

    def one(modality, src):
        src = acquire_source(src, allow_files, processor.opt.max_source_bytes)
        return processor.image(src) if modality == "image" else processor.video(src, fps=video_fps)

    if pool is not None and len(refs) > 1:
        items = pool.map([(lambda m=m, s=s: one(m, s)) for m, s in refs], checkpoint)
    else:
        items = [one(m, s) for m, s in refs]
    return prepare_prompt(tokenizer, rendered_text, items)
