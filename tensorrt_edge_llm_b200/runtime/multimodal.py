"""Multimodal runner: images and audio clips become embedding rows that replace placeholder tokens of the prompt.

The contract of the reference's ``cpp/multimodal/`` runners (``MultimodalRunner`` base and its Qwen-VL style children):
preprocess the media on the host (decode, smart resize, normalise, patchify / log-mel), run the encoder, splice the
rows into the text embeddings where the placeholder token ids sit, compute multimodal RoPE positions when the decoder
uses them, prefill from embeddings, then decode as usual.  Encoders run data-parallel over tensor-parallel ranks and
their outputs are cached by content hash when a cache is given."""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.internvl_vision import InternVisionEncoder, tile_grid
from ..models.qwen_vl_vision import QwenVisionEncoder, patchify_frames
from ..models.vit import EncoderCache, VisionEncoder, dart_prune, encode_data_parallel
from ..ops import reference as ref
from . import native as rt

IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class MultimodalInputs:
    """One request: text pieces and media in the order they appear."""
    pieces: List[Tuple[str, object]] = field(default_factory=list)      # ("text", token ids) | ("image", Image) | ("audio", (samples, rate))

    def text(self, ids: Sequence[int]) -> "MultimodalInputs":
        self.pieces.append(("text", [int(t) for t in ids]))
        return self

    def image(self, image) -> "MultimodalInputs":
        self.pieces.append(("image", image))
        return self

    def video(self, frames: Sequence) -> "MultimodalInputs":
        """A clip as a list of frames (decoded images, arrays, bytes or paths).  It takes the place of one image whose grid
        has a time axis: Qwen-VL towers fold ``temporal_patch_size`` frames into one grid step."""
        self.pieces.append(("image", list(frames)))
        return self

    def audio(self, samples, sample_rate: int) -> "MultimodalInputs":
        self.pieces.append(("audio", (np.asarray(samples, dtype=np.float32), int(sample_rate))))
        return self


@dataclass
class MultimodalPrompt:
    """A prompt ready for the engine: placeholder ids where media sits and the rows actually fed.  Behaves like its id list
    (``len``, iteration), so request plumbing that counts or echoes prompt tokens needs no special case."""
    ids: List[int]
    embeds: torch.Tensor
    positions3: Optional[torch.Tensor] = None
    rope_delta: int = 0
    deepstack: Optional[dict] = None

    def __len__(self) -> int:
        return len(self.ids)

    def __iter__(self):
        return iter(self.ids)


class MultimodalRunner:
    def __init__(self, llm, vision: Optional[VisionEncoder] = None, audio=None, image_token_id: int = 0, audio_token_id: int = 1,
                 cache_bytes: int = 0, visual_keep_ratio: float = 1.0, min_pixels: int = 0, max_pixels: int = 0, max_tiles: int = 12):
        self.llm, self.vision, self.audio = llm, vision, audio
        self.image_token_id, self.audio_token_id = image_token_id, audio_token_id
        self.cache = EncoderCache(cache_bytes) if cache_bytes > 0 else None
        self.keep_ratio = visual_keep_ratio
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.max_tiles = max_tiles                         # InternVL dynamic resolution: tiles per image (a thumbnail comes on top)
        self.device = llm.device
        self._build_lock = threading.Lock()
        self._grids: List[Tuple[int, int, int]] = []      # (t, rows, columns) of each encoded image in language-model tokens
        self._deep: List[torch.Tensor] = []                # deepstack features of the images encoded last (one tensor per level)
        self.deepstack: Optional[dict] = None              # {decoder layer: (prompt rows, features)} of the prompt built last

    @classmethod
    def from_pretrained(cls, llm, model_dir: str, **kw) -> Optional["MultimodalRunner"]:
        """Runner for a vision-language checkpoint directory, or ``None`` when ``config.json`` names no vision tower this
        build has (Qwen2-VL, Qwen2.5-VL, Qwen3-VL and InternVL are built).  The image placeholder id comes from ``image_token_id``."""
        import json
        import os
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
            hf = json.load(f)
        kind = str(hf.get("model_type", ""))
        if "vision_config" in hf and kind == "internvl":
            tower = InternVisionEncoder.from_pretrained(model_dir, device=llm.device, dtype=llm.cfg.dtype)
            return cls(llm, vision=tower, image_token_id=int(hf.get("image_token_id", 151667)), **kw)
        if "vision_config" not in hf or kind not in ("qwen2_vl", "qwen2_5_vl", "qwen3_vl"):
            return None
        tower = QwenVisionEncoder.from_pretrained(model_dir, device=llm.device, dtype=llm.cfg.dtype)
        return cls(llm, vision=tower, image_token_id=int(hf.get("image_token_id", 151655)), **kw)

    # ---- media → rows ------------------------------------------------------------------------------------
    def _image_patches(self, image) -> torch.Tensor:
        """Decode-side preprocessing: resize to the encoder's square input, normalise, cut into patches ``[1, grid², C·P·P]``."""
        c = self.vision.cfg
        if isinstance(image, (bytes, bytearray)):
            image = rt.parse_image(bytes(image))
        elif isinstance(image, str):
            image = rt.load_image(image)
        elif isinstance(image, np.ndarray):
            image = rt.image_from_array(np.ascontiguousarray(image, dtype=np.uint8))
        if (image.width, image.height) != (c.image_size, c.image_size):
            image = rt.resize_bicubic(image, c.image_size, c.image_size)
        chw = torch.from_numpy(rt.normalize_chw(image, list(IMAGE_MEAN), list(IMAGE_STD)))
        return VisionEncoder.patchify(chw[None], c.patch_size)

    def _decode(self, image):
        if isinstance(image, (bytes, bytearray)):
            return rt.parse_image(bytes(image))
        if isinstance(image, str):
            return rt.load_image(image)
        if isinstance(image, np.ndarray):
            return rt.image_from_array(np.ascontiguousarray(image, dtype=np.uint8))
        return image

    def _encode_qwen(self, images: Sequence) -> List[torch.Tensor]:
        """Qwen-VL towers take images at (nearly) their own aspect ratio: sides are rounded to multiples of patch × merge
        inside the pixel budget, and every image brings its own ``(t, h, w)`` grid."""
        c = self.vision.cfg
        factor = c.patch_size * c.spatial_merge_size
        lo = self.min_pixels or 4 * factor * factor
        hi = self.max_pixels or 1280 * factor * factor
        mats, grids = [], []
        for im in images:
            frames = [self._decode(f) for f in (im if isinstance(im, list) else [im])]     # a list is a video clip
            hh, ww = rt.smart_resize(frames[0].height, frames[0].width, factor, lo, max(hi // max(len(frames) // c.temporal_patch_size, 1), lo))
            chw = []
            for f in frames:                                   # every frame of a clip goes to the first frame's size
                if (f.height, f.width) != (hh, ww):
                    f = rt.resize_bicubic(f, ww, hh)
                chw.append(torch.from_numpy(rt.normalize_chw(f, list(IMAGE_MEAN), list(IMAGE_STD))))
            m, g = patchify_frames(torch.stack(chw), c)
            mats.append(m)
            grids.append(g)
        m = c.spatial_merge_size
        self._grids = [(t, h // m, w // m) for t, h, w in grids]
        levels = len(c.deepstack_visual_indexes)
        # encoder cache: one entry per image, the tower's rows and its deepstack levels side by side ([rows, (1 + levels) · H])
        keys = [EncoderCache.key(x) for x in mats] if self.cache is not None else [None] * len(mats)
        packed: List[Optional[torch.Tensor]] = [self.cache.get(k) if self.cache is not None else None for k in keys]
        todo = [i for i, p in enumerate(packed) if p is None]
        if todo:
            res = self.vision(torch.cat([mats[i] for i in todo], 0).to(self.device), [grids[i] for i in todo], return_deepstack=bool(levels))
            rows, deep = res if isinstance(res, tuple) else (res, [])
            at = 0
            for i in todo:
                t, h, w = self._grids[i]
                n = t * h * w
                packed[i] = torch.cat([rows[at:at + n]] + [d[at:at + n] for d in deep], dim=1)
                if self.cache is not None:
                    self.cache.put(keys[i], packed[i])
                at += n
        width = packed[0].shape[1] // (1 + levels)
        # Qwen3-VL: features of intermediate blocks ride along; they join the language model's first layers (deepstack)
        self._deep = [torch.cat([p[:, (k + 1) * width:(k + 2) * width] for p in packed], 0) for k in range(levels)]
        return [p[:, :width] for p in packed]

    def _encode_intern(self, images: Sequence) -> List[torch.Tensor]:
        """InternVL: every image becomes up to ``max_tiles`` square tiles on the grid closest to its aspect ratio, plus a
        thumbnail of the whole image when it was split; the rows of all its tiles follow one another in the prompt."""
        c = self.vision.cfg
        s = c.image_size
        tiles, counts = [], []
        for im in images:
            im = self._decode(im)
            cols, rows = tile_grid(im.width, im.height, s, 1, self.max_tiles)
            big = rt.resize_bicubic(im, cols * s, rows * s)
            chw = torch.from_numpy(rt.normalize_chw(big, list(self.vision.image_mean), list(self.vision.image_std)))
            parts = [chw[:, r * s:(r + 1) * s, q * s:(q + 1) * s] for r in range(rows) for q in range(cols)]
            if len(parts) > 1:
                thumb = rt.resize_bicubic(im, s, s)
                parts.append(torch.from_numpy(rt.normalize_chw(thumb, list(self.vision.image_mean), list(self.vision.image_std))))
            tiles += parts
            counts.append(len(parts))
        out_rows = self.vision(torch.stack(tiles).to(self.device))
        per = out_rows.shape[0] // len(tiles)
        out, at = [], 0
        for n in counts:
            out.append(out_rows[at:at + n * per])
            at += n * per
        return out

    def encode_images(self, images: Sequence) -> List[torch.Tensor]:
        self._grids, self._deep = [], []
        if not images:
            return []
        if self.vision is None:
            raise ValueError("this runner has no vision encoder")
        if any(isinstance(im, list) for im in images) and not isinstance(self.vision, QwenVisionEncoder):
            raise ValueError("video clips need a tower with a time axis (Qwen-VL)")
        if isinstance(self.vision, InternVisionEncoder):
            rows = self._encode_intern(images)
            if self.keep_ratio < 1.0:
                rows = [r[dart_prune(r, max(1, int(round(r.shape[0] * self.keep_ratio))))] for r in rows]
            return rows
        if isinstance(self.vision, QwenVisionEncoder):
            if self.keep_ratio < 1.0:
                raise ValueError("visual-token pruning is not combined with grid-shaped (multimodal RoPE) image rows")
            return self._encode_qwen(images)
        patches = torch.cat([self._image_patches(im) for im in images], 0).to(self.device)
        enc = (lambda x: encode_data_parallel(self.vision, x, self.llm.model.comm))
        rows = self.cache.encode(enc, patches) if self.cache is not None else enc(patches)
        per = rows.shape[0] // len(images)
        out = [rows[i * per:(i + 1) * per] for i in range(len(images))]
        if self.keep_ratio < 1.0:                        # visual-token pruning: near-duplicate rows of an image are dropped
            out = [r[dart_prune(r, max(1, int(round(r.shape[0] * self.keep_ratio))))] for r in out]
        return out

    def encode_audio(self, clips: Sequence[Tuple[np.ndarray, int]]) -> List[torch.Tensor]:
        if not clips:
            return []
        if self.audio is None:
            raise ValueError("this runner has no audio encoder")
        from ..models.audio import audio_features
        c = self.audio.cfg
        seconds = 2 * c.max_source_positions // 100
        out = []
        for samples, rate in clips:
            mel = audio_features(samples, rate, n_mels=c.n_mels, chunk_seconds=seconds).to(self.device)
            out.append(self.cache.encode(self.audio, mel) if self.cache is not None else self.audio(mel))
        return out

    # ---- request → prompt rows ----------------------------------------------------------------------------
    def build(self, req: MultimodalInputs):
        """Token ids with placeholder runs, the embedding rows with media spliced in, and (for multimodal-RoPE decoders)
        the 3-D positions and decode offset."""
        images = self.encode_images([p for k, p in req.pieces if k == "image"])
        clips = self.encode_audio([p for k, p in req.pieces if k == "audio"])
        ids: List[int] = []
        media_rows: List[torch.Tensor] = []
        grids = []
        ii = ai = 0
        for kind, payload in req.pieces:
            if kind == "text":
                ids += payload
            elif kind == "image":
                rows = images[ii]
                ii += 1
                ids += [self.image_token_id] * rows.shape[0]
                media_rows.append(rows)
                side = int(round(rows.shape[0] ** 0.5))
                if self._grids:
                    grids.append(self._grids[ii - 1])
                else:
                    grids.append((1, side, side) if side * side == rows.shape[0] else (1, 1, rows.shape[0]))
            else:
                rows = clips[ai]
                ai += 1
                ids += [self.audio_token_id] * rows.shape[0]
                media_rows.append(rows)
        runner = self.llm.runner
        safe = [t if t not in (self.image_token_id, self.audio_token_id) else 0 for t in ids]
        emb = runner.embed_tokens(safe).clone()
        if media_rows:
            pos = torch.tensor([i for i, t in enumerate(ids) if t in (self.image_token_id, self.audio_token_id)], device=emb.device)
            emb[pos] = torch.cat(media_rows, 0).to(emb.device, emb.dtype)
        self.deepstack = None
        if self._deep and media_rows:
            # level k of the tower's deepstack features is added to the image rows after decoder layer k
            img_pos = torch.tensor([i for i, t in enumerate(ids) if t == self.image_token_id], dtype=torch.int64)
            self.deepstack = {k: (img_pos, f.to(emb.dtype)) for k, f in enumerate(self._deep)}
        positions3 = delta = None
        if self.llm.cfg.mrope_section:
            # audio runs advance like text; image runs use their (t, h, w) grid (rows are already merged: merge factor 1)
            img_only = [t if t != self.audio_token_id else -1 for t in ids]
            positions3, delta = ref.mrope_positions(img_only, self.image_token_id, grids, spatial_merge=1)
        return ids, emb, positions3, delta

    @torch.no_grad()
    def prepare(self, req: MultimodalInputs) -> MultimodalPrompt:
        """Encode the media and build the prompt the request engine takes (``LLM.submit`` / ``LLM.generate`` accept it)."""
        with self._build_lock:
            ids, emb, positions3, delta = self.build(req)
            return MultimodalPrompt(ids, emb, positions3, int(delta or 0), self.deepstack)

    @torch.no_grad()
    def generate(self, req: MultimodalInputs, max_tokens: int = 32, seat: int = 0) -> List[int]:
        with self._build_lock:                 # the encoders keep scratch buffers: one prompt is built at a time
            ids, emb, positions3, delta = self.build(req)
            deep = self.deepstack
        if self.llm.engine is not None:
            # in-flight batching: the request engine owns the seats; the prompt joins its steps next to everyone else's rows
            from .runner import SamplingParams
            h = self.llm.submit_multimodal(ids, emb, SamplingParams(max_tokens=max_tokens, ignore_eos=True), positions3, delta or 0, deep)
            toks = h.get(3600.0)
            if h.error():
                raise RuntimeError(h.error())
            return [int(t) for t in toks]
        runner, kv = self.llm.runner, self.llm.kv
        kv.free(seat)
        kv.reserve(seat, len(ids) + max_tokens)
        logits = runner.prefill_embeds([seat], [emb], positions3=None if positions3 is None else [positions3],
                                       rope_deltas=None if positions3 is None else [delta], deepstack=deep)
        first = runner.pick(logits)
        out = [int(first[0])]
        if max_tokens > 1:
            out += runner.decode_greedy([seat], first, max_tokens - 1)[0].tolist()
        kv.free(seat)
        return out
