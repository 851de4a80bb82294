"""Small Musavik configurations for tests and a writer of model folders of the tests' own.

The shapes differ from one another in everything the configuration can say: the order of the two kinds of
mixer; recurrences of 1 to 5 blocks behind 1 to 4 taps; attention with value heads larger, smaller or equal
to the key size, one to all key heads per query head, rotations over a part, all or none of the head, windows
from a few tokens to more than a page with and without kept first tokens, or no mask; delta rules with one to
all key heads per value head and unlike key and value sizes; the two scales of a pair; layers without a
feed-forward; a loop at the start, in the middle, at the end, run once, or none; a pair table or none; a
width that is no multiple of 8.  Weights are drawn wide enough for attention and gates to be far from uniform.
"""

from __future__ import annotations

import json
import math
import os

import torch


def rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"blocks": blocks, "conv": conv, "width": width}}


def left(heads, kv_heads, dim, vdim, rot, window, keep_first=0, base=10000.0, scale=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim,
         "scale": scale if scale is not None else 6.0 / math.sqrt(dim)}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    if window is not None:
        m["mask"] = {"keep_first": keep_first, "size": window}
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}


def parallel(left_record, right_record, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mixer": {"left": left_record, "left_scale": left_scale, "right": right_record,
                                          "right_scale": right_scale}}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def config(width, vocab, layers, eps=1e-5, embedding_scale=1.0, pairs=None, loop=None):
    """``layers``: (mixer entry, mlp entry or None) pairs; ``pairs``: (buckets, mul_prev, mul_cur) or None;
    ``loop``: (start, stop, times) or None."""
    emb = {"scale": embedding_scale}
    if pairs is not None:
        emb["bigram"] = {"buckets": pairs[0], "mul_cur": pairs[2], "mul_prev": pairs[1]}
    out = {"architecture": "Musavik", "embedding": emb, "layers": [dict(m, mlp=f) for m, f in layers],
           "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# a pair first, looped three times from the start; value heads smaller than keys; a short window with kept
# tokens; a layer without feed-forward; one block; one tap
EARLY = config(96, 211, [
    (parallel(left(4, 2, 24, 16, 12, 9, keep_first=3), right(4, 2, 16, 24, 2), 0.7, 1.3), dense(80)),
    (rglru(64, 1, 1), None),
    (rglru(80, 5, 4), dense(56))], embedding_scale=2.0, pairs=(97, 31, 7), loop=(0, 2, 3))
# no loop and no pair table; every query head its own key head, the whole head rotated, a window of more than
# a page; equal key and value sizes
FLAT = config(128, 157, [
    (rglru(96, 3, 2), dense(72)),
    (parallel(left(3, 3, 32, 32, 32, 70, keep_first=5, base=500.0), right(3, 3, 32, 32, 4), 1.0, 0.25), dense(64)),
    (rglru(128, 4, 3), dense(40))], eps=1e-6, embedding_scale=0.5)
# a width no product kernel takes; all query heads on one key head; no rotation in one pair, no mask in the
# other; the loop at the end, run once; multipliers larger than the table
ODD = config(100, 89, [
    (rglru(60, 2, 3), dense(36)),
    (parallel(left(6, 1, 20, 28, 0, 64, keep_first=64), right(6, 1, 12, 20, 3), 0.9, 0.9), None),
    (parallel(left(2, 2, 16, 16, 8, None, base=1e6), right(2, 1, 20, 12, 1), 1.5, 0.5), dense(44))],
    eps=1e-4, embedding_scale=1.5, pairs=(13, 1000, 999), loop=(2, 3, 1))
# key size 128; a loop in the middle; pairs only
WIDE = config(256, 301, [
    (parallel(left(8, 4, 128, 64, 64, 33, keep_first=9, base=2e5), right(4, 2, 64, 32, 4), 0.6, 0.4), dense(96)),
    (parallel(left(4, 1, 64, 128, 16, 130, keep_first=1), right(2, 2, 128, 64, 2), 1.0, 1.0), dense(64)),
    (rglru(192, 2, 4), dense(128))], embedding_scale=3.0, pairs=(499, 3, 5), loop=(1, 2, 2))

SHAPES = {"early": EARLY, "flat": FLAT, "odd": ODD, "wide": WIDE}


def tensor_shapes(cfg):
    w, v = cfg["width"], cfg["vocab"]
    shapes = {"embed": (v, w), "final.norm": (w,), "head": (v, w)}
    if cfg["embedding"].get("bigram"):
        shapes["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, w)
    if cfg.get("loop"):
        shapes["loop.in"] = (w, 2 * w)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        shapes.update({p + "norm1": (w,), p + "norm1b": (w,)})
        if layer["type"] == "rglru":
            r, nb, k = m["width"], m["blocks"], m["conv"]
            s = r // nb
            shapes.update({p + "mix.y": (r, w), p + "mix.y.b": (r,), p + "mix.x": (r, w), p + "mix.x.b": (r,),
                           p + "mix.conv": (r, k), p + "mix.conv.b": (r,), p + "mix.ra": (nb, s, s),
                           p + "mix.ra.b": (nb, s), p + "mix.ri": (nb, s, s), p + "mix.ri.b": (nb, s),
                           p + "mix.lam": (r,), p + "mix.o": (w, r)})
        else:
            a, q = m["left"], p + "mix.left."
            h, g, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            shapes.update({q + "q": (h * d, w), q + "q.b": (h * d,), q + "k": (g * d, w), q + "k.b": (g * d,),
                           q + "v": (g * e, w), q + "v.b": (g * e,), q + "q.norm": (d,), q + "k.norm": (d,),
                           q + "talk": (h, h), q + "g": (h * e, w), q + "o": (w, h * e)})
            b, q = m["right"], p + "mix.right."
            h, g, d, e, k = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
            shapes.update({q + "q": (g * d, w), q + "q.conv": (g * d, k), q + "k": (g * d, w), q + "k.conv": (g * d, k),
                           q + "v": (h * e, w), q + "v.conv": (h * e, k), q + "b": (h, w), q + "A_log": (h,),
                           q + "norm": (e,), q + "a": (h, w), q + "dt_bias": (h,), q + "g": (h * e, w),
                           q + "o": (w, h * e)})
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "norm2": (w,), p + "norm2b": (w,), p + "mlp.up": (ff, w), p + "mlp.up.b": (ff,),
                           p + "mlp.down": (w, ff), p + "mlp.down.b": (w,)})
    return shapes


def make_tensors(cfg, seed, dtype=torch.bfloat16):
    """Matrices N(0, 1/in); norm weights around zero (the model adds the 1), the two head norms around 1; biases
    a few tenths; decay rates spread over two decades; a head mix with a strong diagonal and some negative
    entries."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        t = torch.randn(shape, generator=g, dtype=torch.float32)
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("q.norm", "k.norm", "right.norm")):
            t = 1.0 + 0.2 * t
        elif last in ("norm", "norm1", "norm1b", "norm2", "norm2b"):
            t = 0.2 * t
        elif last == "talk":
            t = torch.eye(shape[0]) + 0.4 * t
        elif last == "conv":
            t = 0.6 * t
        elif last == "b" and len(shape) <= 2 and not name.endswith("right.b"):
            t = 0.3 * t                          # biases (also the gates' [blocks, size])
        elif last == "lam":
            t = 1.5 * t - 2.0
        elif last == "A_log":
            t = 1.5 * t - 1.0
        elif last == "dt_bias":
            t = t - 1.0
        elif name in ("embed", "bigram"):
            pass
        elif last in ("ra", "ri"):
            t = t * (2.0 / math.sqrt(shape[-1]))
        else:
            t = t / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


def write_folder(folder, cfg, tensors):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def random_prompts(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]
