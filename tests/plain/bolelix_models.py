"""Small Bolelix configurations for tests and a writer of model folders of the tests' own.

The shapes differ from one another in everything the configuration can say: the order of the three
mixers; attention with value heads larger, smaller or equal to the key size, one to all key heads per
query head, rotations over a part or all of the head with and without divided frequencies, windows from
a few tokens to more than a page with and without kept first tokens, layers that read an earlier layer's
keys through a window of their own; state-space layers with one group to one per head, 1 to 5 taps, the
norm in one part or several; matrix memories with unlike key and value sizes; routers choosing 1 to 6 of
2 to 16 experts; layers without a feed-forward; a width that is no multiple of 8.  Weights are drawn wide
enough for attention, gates and routing to be far from uniform.
"""

from __future__ import annotations

import json
import math
import os

import torch


def attention(heads, kv_heads, dim, vdim, rot, window, keep_first=0, factor=None, base=10000.0, scale=None,
              kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim,
         "scale": scale if scale is not None else 6.0 / math.sqrt(dim)}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    if window is not None:
        m["mask"] = {"keep_first": keep_first, "size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def mamba2(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups,
                                        "state": state, "vdim": vdim}}


def mlstm(heads, dim, vdim, cap=15.0):
    return {"type": "mlstm", "mixer": {"dim": dim, "gate_cap": cap, "heads": heads, "vdim": vdim}}


def moe(experts, ff, top):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}


def config(width, vocab, layers, eps=1e-5, embedding_scale=1.0):
    """``layers``: (mixer entry, mlp entry or None) pairs."""
    return {"architecture": "Bolelix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embedding_scale}, "layers": [dict(m, mlp=f) for m, f in layers]}


# attention first, value heads larger than keys, a short window with kept tokens; a later layer reads its keys
# through another window and keeps none; a layer without feed-forward
MIXED = config(96, 211, [
    (attention(4, 2, 24, 40, 16, 9, keep_first=3, factor=2.0), moe(8, 48, 2)),
    (mamba2(4, 16, 24, 2, 3, 4), moe(5, 40, 3)),
    (mlstm(3, 20, 12, cap=10.0), None),
    (attention(4, 2, 24, 40, 16, 17, factor=2.0, kv_from=0), moe(6, 32, 1))], embedding_scale=2.0)
# recurrences first; every query head its own key head, the whole head rotated, plain frequencies, a window
# of more than a page; one group per head; one tap
PLAIN = config(128, 157, [
    (mlstm(2, 64, 32), moe(6, 40, 3)),
    (mamba2(2, 32, 16, 2, 1, 1), None),
    (attention(3, 3, 32, 32, 32, 70, keep_first=5, base=500.0), moe(4, 56, 2))], eps=1e-6, embedding_scale=0.5)
# a width no product kernel takes; value heads smaller than keys; all query heads on one key head; a window
# of one page exactly; two layers reading the same earlier keys; five taps; no mask at all in one layer
ODD = config(100, 89, [
    (mamba2(6, 10, 40, 1, 5, 3), moe(2, 36, 2)),
    (attention(6, 1, 40, 12, 10, 64, keep_first=64, factor=8.0, base=1e6), None),
    (attention(6, 1, 40, 12, 10, 3, keep_first=1, factor=8.0, base=1e6, kv_from=1), moe(3, 20, 1)),
    (attention(6, 1, 40, 12, 10, 30, keep_first=2, factor=8.0, base=1e6, kv_from=1), moe(3, 20, 3)),
    (attention(2, 2, 16, 16, 0, None), None),
    (mlstm(5, 12, 20, cap=4.0), moe(7, 24, 4))], eps=1e-4, embedding_scale=1.5)
# key size 128, state 128, many experts
WIDE = config(256, 301, [
    (mamba2(4, 64, 128, 2, 4, 2), moe(16, 32, 6)),
    (attention(8, 4, 128, 64, 64, 33, keep_first=9, factor=4.0), moe(12, 64, 1)),
    (mlstm(2, 128, 64), moe(4, 48, 2))], embedding_scale=3.0)

SHAPES = {"mixed": MIXED, "plain": PLAIN, "odd": ODD, "wide": WIDE}


def tensor_shapes(cfg):
    w, v = cfg["width"], cfg["vocab"]
    shapes = {"embed": (v, w), "final.norm": (w,), "head": (v, w)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        shapes.update({p + "norm1": (w,), p + "ls1": (w,)})
        if layer["type"] == "attention":
            h, g, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (h * d, w), p + "mix.g": (h, w), p + "mix.o": (w, h * e)})
            if m.get("kv_from") is None:
                shapes.update({p + "mix.k": (g * d, w), p + "mix.v": (g * e, w)})
        elif layer["type"] == "mamba2":
            h, e, n, g, k = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = h * e, h * e + 2 * g * n
            shapes.update({p + "mix.in": (2 * inner + 2 * g * n + h, w), p + "mix.conv": (ch, k), p + "mix.conv.b": (ch,),
                           p + "mix.dt_bias": (h,), p + "mix.A_log": (h,), p + "mix.D": (h,), p + "mix.norm": (inner,),
                           p + "mix.o": (w, inner)})
        else:
            h, d, e = m["heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (h * d, w), p + "mix.k": (h * d, w), p + "mix.v": (h * e, w), p + "mix.g": (h * e, w),
                           p + "mix.i": (h, w), p + "mix.i.b": (h,), p + "mix.f": (h, w), p + "mix.f.b": (h,),
                           p + "mix.norm": (h * e,), p + "mix.o": (w, h * e)})
        mlp = layer["mlp"]
        if mlp is not None:
            shapes[p + "ls2"] = (w,)
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], w)
            for e in range(mlp["router"]["experts"]):
                ff = mlp["expert"]["ff"]
                shapes.update({f"{p}mlp.e{e}.gate": (ff, w), f"{p}mlp.e{e}.up": (ff, w), f"{p}mlp.e{e}.down": (w, ff)})
    return shapes


def make_tensors(cfg, seed, dtype=torch.bfloat16, sharp=1.0):
    """Matrices N(0, 1/in); gains and layer scales around 1 (some negative); decay rates spread over two decades;
    gate biases that keep some memory; ``sharp`` multiplies the routers (and, below 1, its square the experts'
    output)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        t = torch.randn(shape, generator=g, dtype=torch.float32)
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "D"):
            t = 1.0 + 0.2 * t
        elif last in ("ls1", "ls2"):
            t = 0.7 + 0.3 * t
        elif last == "conv":
            t = 0.6 * t
        elif name.endswith("conv.b"):
            t = 0.2 * t
        elif last == "A_log":
            t = 1.5 * t - 1.0
        elif last == "dt_bias":
            t = t - 1.0
        elif name.endswith(".i.b"):
            t = t
        elif name.endswith(".f.b"):
            t = t + 3.0
        elif name == "embed":
            pass
        else:
            t = t / math.sqrt(shape[1])
            if last == "router":
                t = t * 1.5 * sharp
            if last in ("i", "f"):
                t = t * 2.0
            if ".mlp.e" in name and last == "down" and sharp < 1.0:
                t = t * sharp * sharp            # mild weights: a token sent to another expert moves little
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
