"""Vision tower of the Qwen3-VL / Qwen3.5 family and the image pre-processing that feeds it.

An image becomes a grid of 16 x 16 patches (each repeated over two "frames"); the tower embeds the patches (a strided 3-D
convolution, evaluated as one GEMM over the flattened patches), adds a learned position table interpolated to the grid,
runs ``depth`` pre-norm blocks of full (non-causal) attention with a 2-D rotary embedding over (row, column), and merges every
2 x 2 block of patches into one token of the language model's width.  The language model sees those tokens in place of its
image placeholder tokens, with (time, row, column) rotary positions (``mrope_positions`` / ``mrope_tables`` below).

Reference: the vision path of src/models/qwen3_5.cpp (Qwen3_5Model::VisionForward, the ``visual.*`` weights) and the image
pre-processing of tools/fastllm_pytools (smart resize to multiples of patch x merge, mean / std 0.5).
"""
from __future__ import annotations

import base64
import io
import math

import torch
import torch.nn.functional as F


class VisionConfig:
    def __init__(self, d: dict):
        g = d.get
        self.depth = int(g("depth", 27))
        self.hidden = int(g("hidden_size", 1152))
        self.inter = int(g("intermediate_size", 4304))
        self.heads = int(g("num_heads", 16))
        self.in_ch = int(g("in_channels", 3))
        self.patch = int(g("patch_size", 16))
        self.merge = int(g("spatial_merge_size", 2))
        self.t_patch = int(g("temporal_patch_size", 2))
        self.out_hidden = int(g("out_hidden_size", 3584))
        self.num_pos = int(g("num_position_embeddings", 2304))
        self.act = g("hidden_act", "gelu_pytorch_tanh")
        self.deepstack = list(g("deepstack_visual_indexes", []) or [])


class VisionTower:
    """Weights (``visual.*``) and forward pass; runs in ``dtype`` on ``device`` with PyTorch ops (the tower runs once per
    image, not per generated token)."""

    def __init__(self, cfg: VisionConfig, weights: dict, device, dtype):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(self.device, dtype) for k, v in weights.items()}
        if self.cfg.deepstack:
            raise NotImplementedError("deep-stack visual features (Qwen3-VL) are not merged into the decoder layers")

    def _lin(self, x, name):
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _pos_embed(self, grids):
        """Learned position table (a square grid) interpolated bilinearly to every image's patch grid, in merge-block order."""
        c = self.cfg
        side = int(c.num_pos ** 0.5)
        table = self.w["pos_embed.weight"].float()
        out = []
        for t, h, w in grids:
            hi, wi = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
            h0, w0 = hi.int(), wi.int()
            h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
            dh, dw = (hi - h0)[:, None], (wi - w0)[None, :]
            idx = lambda a, b: (a[:, None] * side + b[None, :]).reshape(-1).long().to(table.device)
            wt = lambda m: m.reshape(-1, 1).to(table.device)
            pe = (table[idx(h0, w0)] * wt((1 - dh) * (1 - dw)) + table[idx(h0, w1)] * wt((1 - dh) * dw)
                  + table[idx(h1, w0)] * wt(dh * (1 - dw)) + table[idx(h1, w1)] * wt(dh * dw))
            pe = pe.repeat(t, 1).view(t, h // c.merge, c.merge, w // c.merge, c.merge, -1).permute(0, 1, 3, 2, 4, 5).reshape(t * h * w, -1)
            out.append(pe)
        return torch.cat(out).to(self.dtype)

    def _rotary(self, grids):
        c = self.cfg
        hd = c.hidden // c.heads
        dim = hd // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        rows = []
        for t, h, w in grids:
            mh, mw, m = h // c.merge, w // c.merge, c.merge
            r = (torch.arange(mh)[:, None, None, None] * m + torch.arange(m)[None, None, :, None]).expand(mh, mw, m, m).reshape(-1)
            cc = (torch.arange(mw)[None, :, None, None] * m + torch.arange(m)[None, None, None, :]).expand(mh, mw, m, m).reshape(-1)
            fr = torch.cat([r[:, None].float() * inv[None, :], cc[:, None].float() * inv[None, :]], dim=-1)     # [h*w, hd/2]
            rows.append(fr.repeat(t, 1))
        fr = torch.cat(rows).to(self.device)
        emb = torch.cat([fr, fr], dim=-1)
        return emb.cos(), emb.sin()

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grids) -> torch.Tensor:
        """``patches`` ``[sum(t*h*w), in_ch * t_patch * patch * patch]`` in merge-block order, ``grids`` list of (t, h, w) in
        patches -> ``[sum(t*h*w) / merge^2, out_hidden]``."""
        c = self.cfg
        x = patches.to(self.device, self.dtype)
        h = F.linear(x, self.w["patch_embed.proj.weight"].reshape(c.hidden, -1), self.w.get("patch_embed.proj.bias"))
        h = h + self._pos_embed(grids)
        cos, sin = self._rotary(grids)
        S = h.shape[0]
        hd = c.hidden // c.heads
        bounds = [0]
        for t, gh, gw in grids:
            for _ in range(t):
                bounds.append(bounds[-1] + gh * gw)           # attention stays inside one frame
        for i in range(c.depth):
            p = f"blocks.{i}."
            y = F.layer_norm(h, (c.hidden,), self.w[p + "norm1.weight"], self.w[p + "norm1.bias"], 1e-6)
            q, k, v = self._lin(y, p + "attn.qkv").reshape(S, 3, c.heads, hd).permute(1, 0, 2, 3).unbind(0)
            rot = lambda t_: torch.cat([-t_[..., hd // 2:], t_[..., :hd // 2]], dim=-1)
            qf, kf = q.float(), k.float()
            q = (qf * cos[:, None, :] + rot(qf) * sin[:, None, :]).to(self.dtype)
            k = (kf * cos[:, None, :] + rot(kf) * sin[:, None, :]).to(self.dtype)
            outs = []
            for a, b in zip(bounds[:-1], bounds[1:]):
                o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None], v[a:b].transpose(0, 1)[None])
                outs.append(o[0].transpose(0, 1).reshape(b - a, c.hidden))
            h = h + self._lin(torch.cat(outs), p + "attn.proj")
            y = F.layer_norm(h, (c.hidden,), self.w[p + "norm2.weight"], self.w[p + "norm2.bias"], 1e-6)
            y = self._lin(y, p + "mlp.linear_fc1")
            y = F.gelu(y, approximate="tanh") if "tanh" in c.act else F.gelu(y)
            h = h + self._lin(y, p + "mlp.linear_fc2")
        y = F.layer_norm(h, (c.hidden,), self.w["merger.norm.weight"], self.w["merger.norm.bias"], 1e-6).view(-1, c.hidden * c.merge ** 2)
        return self._lin(F.gelu(self._lin(y, "merger.linear_fc1")), "merger.linear_fc2")


# ---------------------------------------------------------------------------------------------------
# image -> patches
# ---------------------------------------------------------------------------------------------------
def smart_resize(height: int, width: int, factor: int, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
    """Target size: both sides multiples of ``factor``, the area within [min_pixels, max_pixels], the aspect ratio kept."""
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def load_image(src):
    """PIL image from a PIL image, a path, raw bytes or a ``data:image/...;base64,`` URL."""
    from PIL import Image

    if hasattr(src, "convert"):
        return src.convert("RGB")
    if isinstance(src, (bytes, bytearray)):
        return Image.open(io.BytesIO(src)).convert("RGB")
    s = str(src)
    if s.startswith("data:"):
        return Image.open(io.BytesIO(base64.b64decode(s.split(",", 1)[1]))).convert("RGB")
    if s.startswith("file://"):
        s = s[7:]
    if s.startswith("http://") or s.startswith("https://"):
        raise ValueError("remote image URLs are not fetched: pass a file path or a data: URL")
    return Image.open(s).convert("RGB")


def image_to_patches(img, cfg: VisionConfig, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5), min_pixels=None, max_pixels=None):
    """One image -> (``[h*w, in_ch * t_patch * patch * patch]`` fp32 patches in merge-block order, grid ``(1, h, w)``)."""
    from PIL import Image

    img = load_image(img)
    f = cfg.patch * cfg.merge
    kw = {}
    if min_pixels:
        kw["min_pixels"] = min_pixels
    if max_pixels:
        kw["max_pixels"] = max_pixels
    H, W = smart_resize(img.height, img.width, f, **kw)
    img = img.resize((W, H), Image.BICUBIC)
    x = torch.frombuffer(bytearray(img.tobytes()), dtype=torch.uint8).view(H, W, 3).permute(2, 0, 1).float() / 255.0
    x = (x - torch.tensor(mean)[:, None, None]) / torch.tensor(std)[:, None, None]
    return pixels_to_patches(x, cfg)


def pixels_to_patches(x: torch.Tensor, cfg: VisionConfig):
    """``x`` ``[3, H, W]`` normalised pixels (H, W multiples of patch x merge) -> (patches, grid)."""
    C, H, W = x.shape
    p, m, tp = cfg.patch, cfg.merge, cfg.t_patch
    gh, gw = H // p, W // p
    x = x[None].repeat(tp, 1, 1, 1)                                          # the still image fills every temporal slot
    x = x.view(tp, C, gh // m, m, p, gw // m, m, p).permute(2, 5, 3, 6, 1, 0, 4, 7)     # block row, block col, in-block row / col, C, T, p, p
    return x.reshape(gh * gw, C * tp * p * p).contiguous(), (1, gh, gw)


# ---------------------------------------------------------------------------------------------------
# videos: frames in groups of the tower's temporal patch size; every group is laid out like one image and the prompt
# carries a time stamp in front of each (reference: the Qwen3.5 multimodal pre-processing of the server,
# tools/fastllm_pytools/qwen35_multimodal.py; transformers' Qwen3-VL video processor has the same layout)
# ---------------------------------------------------------------------------------------------------
def load_video(src, target_fps: float = 2.0, min_frames: int = 4, max_frames: int = 64):
    """A video -> (sampled frames as PIL images, their time stamps in seconds).  ``src``: a list of frames (paths, bytes,
    ``data:`` URLs, PIL images), a dict ``{"frames": [...], "fps": f}``, a directory of frame images, an animated GIF / WebP /
    PNG (path, bytes or ``data:`` URL), or any container OpenCV can read when ``cv2`` is installed.  Frames are sampled
    uniformly at about ``target_fps`` within ``[min_frames, max_frames]``."""
    import os

    fps = None
    if isinstance(src, dict):
        fps = src.get("fps")
        src = src.get("frames")
    frames = None
    if isinstance(src, (list, tuple)):
        frames = [load_image(f).convert("RGB") for f in src]
    elif isinstance(src, str) and os.path.isdir(src):
        names = sorted(n for n in os.listdir(src) if n.lower().rsplit(".", 1)[-1] in ("png", "jpg", "jpeg", "bmp", "webp"))
        frames = [load_image(os.path.join(src, n)).convert("RGB") for n in names]
    else:
        try:
            from PIL import ImageSequence

            im = load_image(src)
            if getattr(im, "n_frames", 1) > 1:
                dur = im.info.get("duration")
                fps = 1000.0 / dur if dur else fps
                frames = [f.convert("RGB") for f in ImageSequence.Iterator(im)]
        except Exception:
            frames = None
        if frames is None and isinstance(src, str) and os.path.exists(src):
            try:
                import cv2
            except ImportError as e:
                raise ValueError("this video container needs OpenCV (cv2), which is not installed: pass the frames, a frame "
                                 "directory or an animated GIF / WebP instead") from e
            from PIL import Image

            cap = cv2.VideoCapture(src)
            fps = cap.get(cv2.CAP_PROP_FPS) or fps
            frames = []
            while True:
                ok, fr = cap.read()
                if not ok:
                    break
                frames.append(Image.fromarray(cv2.cvtColor(fr, cv2.COLOR_BGR2RGB)))
            cap.release()
    if not frames:
        raise ValueError("no frames could be read from the video input")
    fps = float(fps) if fps else target_fps
    n = len(frames)
    want = int(round(n / fps * target_fps)) if fps > 0 else n
    want = max(min(min_frames, n), min(want, max_frames, n))
    idx = [int(round(i * (n - 1) / max(1, want - 1))) for i in range(want)] if want > 1 else [0]
    return [frames[i] for i in idx], [i / fps for i in idx]


def frames_to_patches(frames, times, cfg: VisionConfig, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5), min_pixels=None, max_pixels=None):
    """Sampled frames -> one ``(patches, grid (1, h, w), time stamp)`` per temporal group of ``cfg.t_patch`` frames (the last
    frame is repeated to fill the last group).  A group's patches hold its frames in the temporal slots, so the rows equal
    one ``(t, h, w)`` video grid cut along ``t``."""
    from PIL import Image

    tp = cfg.t_patch
    frames, times = list(frames), list(times)
    while len(frames) % tp:
        frames.append(frames[-1])
        times.append(times[-1])
    f = cfg.patch * cfg.merge
    kw = {}
    if min_pixels:
        kw["min_pixels"] = min_pixels
    if max_pixels:
        kw["max_pixels"] = max_pixels
    H, W = smart_resize(frames[0].height, frames[0].width, f, **kw)
    px = []
    for im in frames:
        im = im.resize((W, H), Image.BICUBIC)
        x = torch.frombuffer(bytearray(im.tobytes()), dtype=torch.uint8).view(H, W, 3).permute(2, 0, 1).float() / 255.0
        px.append((x - torch.tensor(mean)[:, None, None]) / torch.tensor(std)[:, None, None])
    p, m = cfg.patch, cfg.merge
    gh, gw = H // p, W // p
    out = []
    for g in range(0, len(px), tp):
        x = torch.stack(px[g:g + tp])                                        # [tp, C, H, W]
        x = x.view(tp, 3, gh // m, m, p, gw // m, m, p).permute(2, 5, 3, 6, 1, 0, 4, 7)
        out.append((x.reshape(gh * gw, 3 * tp * p * p).contiguous(), (1, gh, gw), sum(times[g:g + tp]) / tp))
    return out


def video_markup(groups) -> str:
    """Prompt text of one video: a time stamp and one placeholder run per temporal group."""
    return "".join(f"<{t:.1f} seconds>{VIDEO_MARKER}" for _p, _g, t in groups)


# ---------------------------------------------------------------------------------------------------
# (time, row, column) rotary positions of a prompt with images
# ---------------------------------------------------------------------------------------------------
def mrope_positions(ids, image_token_id, grids, merge: int):
    """3-D positions ``[3, T]`` for a prompt whose image placeholder runs (one per image, ``t*h*w / merge^2`` tokens each) are
    laid out on their (time, row, column) grids; text tokens advance all three axes together.  Also returns the offset between
    the next token's position and the sequence length (reference semantics: Qwen2-VL ``get_rope_index``)."""
    T = len(ids)
    pos = torch.zeros((3, T), dtype=torch.long)
    nxt, i, gi = 0, 0, 0
    marks = set(image_token_id) if isinstance(image_token_id, (set, frozenset, list, tuple)) else {image_token_id}
    while i < T:
        if ids[i] in marks and gi < len(grids):
            t, h, w = grids[gi]
            gh, gw = h // merge, w // merge
            n = t * gh * gw
            pos[0, i:i + n] = nxt
            pos[1, i:i + n] = nxt + torch.arange(gh).repeat_interleave(gw).repeat(t)
            pos[2, i:i + n] = nxt + torch.arange(gw).repeat(gh * t)
            nxt += max(gh, gw)
            i += n
            gi += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos, nxt - T


def mrope_tables(pos3: torch.Tensor, rot_dim: int, theta: float, sections, device="cpu"):
    """Per-token (cos, sin) rows ``[T, rot_dim / 2]``: frequency j takes its angle from the time axis, except the interleaved
    slots ``1, 4, 7, ... < 3 * sections[1]`` (row axis) and ``2, 5, 8, ... < 3 * sections[2]`` (column axis)."""
    half = rot_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    axis = torch.zeros(half, dtype=torch.long)
    axis[1:3 * sections[1]:3] = 1
    axis[2:3 * sections[2]:3] = 2
    ang = pos3.double()[axis, :].t() * inv[None, :]                          # [T, half]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


# ---------------------------------------------------------------------------------------------------
# prompts with images
# ---------------------------------------------------------------------------------------------------
IMAGE_MARKER = "<|vision_start|><|image_pad|><|vision_end|>"
VIDEO_MARKER = "<|vision_start|><|video_pad|><|vision_end|>"


def video_slot(k: int) -> str:
    """Stand-in for the k-th video of a conversation until its frames are read and its markup is known."""
    return f"\x00video{k}\x00"


def video_source(part: dict):
    t = part.get("type")
    if t == "video_url":
        u = part.get("video_url")
        return u.get("url") if isinstance(u, dict) else u
    if t in ("video", "input_video"):
        return part.get("video") or part.get("video_url") or part.get("url") or part.get("path") or part.get("frames")
    return None


def image_source(part: dict):
    """The image of one content part in the OpenAI (``image_url``), Responses (``input_image``) or Qwen (``image``) form."""
    t = part.get("type")
    if t == "image_url":
        u = part.get("image_url")
        return u.get("url") if isinstance(u, dict) else u
    if t == "input_image":
        return part.get("image_url") or part.get("file_id")
    if t == "image":
        return part.get("image") or part.get("url") or part.get("path")
    return None


def extract_images(messages, videos: list | None = None):
    """Chat messages whose content lists hold image parts -> (messages with plain-text content, every image replaced by the
    placeholder markup of the Qwen-VL chat format, the images in prompt order).  With a ``videos`` list, ``video_url`` /
    ``video`` parts are appended to it and leave ``video_slot(k)`` in the text (without one they are an error)."""
    out, images = [], []
    for m in messages:
        d = dict(m)
        c = d.get("content")
        if isinstance(c, list):
            text = ""
            for part in c:
                if not isinstance(part, dict):
                    continue
                src = image_source(part)
                vsrc = video_source(part) if src is None else None
                if src is not None:
                    images.append(src)
                    text += IMAGE_MARKER
                elif vsrc is not None:
                    if videos is None:
                        raise ValueError("video inputs are not accepted on this route")
                    text += video_slot(len(videos))
                    videos.append(vsrc)
                elif part.get("type", "text") in ("text", "input_text", "output_text"):
                    text += part.get("text", "")
            d["content"] = text
        out.append(d)
    return out, images


def build_context(model, ids, images, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5), min_pixels=None, max_pixels=None, videos=None):
    """Token ids with one placeholder token per image -> (ids with every placeholder repeated once per merged patch, the
    request's ``MultimodalContext``: the tower's embeddings for those tokens and the 3-D rotary positions).  ``videos``: per
    video the temporal groups of ``frames_to_patches``; the ids hold one video placeholder token per group."""
    from ..engine.engine import MultimodalContext

    if getattr(model.cfg, "model_type", "") == "cogvlm":
        from . import cogvlm

        return cogvlm.build_context(model, ids, images)
    tower = getattr(model, "vision", None)
    tok = getattr(model, "image_token_id", None)
    if tower is None or tok is None:
        raise ValueError("this model has no vision tower: image inputs are not supported")
    cfg = tower.cfg
    vtok = getattr(model, "video_token_id", None)
    stills = [image_to_patches(im, cfg, mean, std, min_pixels, max_pixels) for im in images]
    groups = [(p, g) for vid in (videos or []) for p, g, _t in vid]
    if groups and vtok is None:
        raise ValueError("this checkpoint names no video placeholder token: video inputs are not supported")
    patches, grids, out, k, kv = [], [], [], 0, 0        # media in prompt order, images and video groups interleaved
    for t in ids:
        if t == tok and k < len(stills):
            p, g = stills[k]
            k += 1
        elif vtok is not None and t == vtok and kv < len(groups):
            p, g = groups[kv]
            kv += 1
        else:
            out.append(t)
            continue
        patches.append(p)
        grids.append(g)
        out.extend([t] * (g[0] * g[1] * g[2] // cfg.merge ** 2))
    if k != len(stills) or kv != len(groups):
        raise ValueError(f"the prompt holds {k} image and {kv} video-frame placeholders for {len(stills)} images and {len(groups)} video frame groups")
    embeds = tower.forward(torch.cat(patches), grids)
    marks = {tok} if vtok is None else {tok, vtok}
    pos3, delta = mrope_positions(out, marks, grids, cfg.merge)
    at = [i for i, t in enumerate(out) if t in marks][:embeds.shape[0]]
    return out, MultimodalContext(embeds, at, pos3, delta)
