"""Plain, slow restatement of the Zefenex design in float64 on the CPU, one function per mechanism, written from the design's equations
and sharing nothing with the package: the oracle for tests/test_zefenex*.py.

Notation: h is a [T, width] block of one sequence's tokens at positions 0..T-1; W['name'] are float64 tensors, matrices stored [out, in].
Every function sees the WHOLE sequence at once (no cache carried between calls): whatever the engine does with pages, portions and
batches must reproduce these numbers."""
import math

import numpy as np
import torch

F = torch.float64


def dyt(x, W, name):
    """Dynamic Tanh: no mean, no variance."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate(v, positions, base, dims):
    """v [T, ..., n]: the first `dims` of the last axis turn, dimension i together with i + dims/2, by the angle p * base^(-2i/dims)."""
    half = dims // 2
    out = v.clone()
    for i in range(half):
        a = positions.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(a), torch.sin(a)
        while c.dim() < v.dim() - 1:
            c, s = c.unsqueeze(-1), s.unsqueeze(-1)
        u, w = v[..., i], v[..., i + half]
        out[..., i] = u * c - w * s
        out[..., i + half] = w * c + u * s
    return out


def latent_rows(h, W, p, mx, eps):
    """What a layer caches per position: the normed latent row c [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    r = mx["kv_rank"]
    down = h @ W[p + "dkv"].T
    c = rms_unit(down[:, :r], eps) * W[p + "dkv.norm"]
    kr = rotate(down[:, r:], torch.arange(h.shape[0]), mx["rot"]["base"], mx["rot"]["dims"])
    return c, kr


def visible(T, window):
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    return (d >= 0) & ((d < window) if window else torch.ones_like(d, dtype=torch.bool))


def mixer_latent(h, W, p, mx, eps, rows):
    """rows = (c, kr) of this layer or of the layer it borrows from."""
    T = h.shape[0]
    H, d, dr, dv = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"]
    c, kr = rows
    q = (h @ W[p + "q"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], torch.arange(T), mx["rot"]["base"], mx["rot"]["dims"])
    k = (c @ W[p + "uk"].T).view(T, H, d)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    see = visible(T, (mx.get("mask") or {}).get("size", 0))
    heads = []
    for a in range(H):
        s = (q_plain[:, a] @ k[:, a].T + q_rot[:, a] @ kr.T) * mx["scale"]
        e = torch.where(see, torch.exp(s), torch.zeros_like(s))
        denom = e.sum(-1, keepdim=True) + torch.exp(W[p + "sink"][a])   # the sink: in the denominator only
        heads.append((e / denom) @ v[:, a])
    o = torch.cat(heads, -1) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def feed_forward_dense(h, W, p):
    return (torch.relu(h @ W[p + "up"].T + W[p + "up.b"]) ** 2) @ W[p + "down"].T + W[p + "down.b"]


def gated_expert(x, W, p):
    g = x @ W[p + "gate"].T
    return (g * torch.sigmoid(g) * (x @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, ml):
    """-> chosen [T, top] (indices into experts + identity), weight [T, top]."""
    s = torch.softmax(h @ W[p + "router"].T, -1)
    _, chosen = torch.topk(s + W[p + "correction"], ml["router"]["top"], dim=-1)
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20)


def feed_forward_moe(h, W, p, ml):
    chosen, weight = route(h, W, p, ml)
    E = ml["router"]["experts"]
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weight[t]):
            y[t] += w * (h[t] if e >= E else gated_expert(h[t], W, f"{p}e{e}."))   # past the real experts: identity
    if ml.get("shared"):
        y = y + gated_expert(h, W, p + "shared.")
    return y


def forward(config, W, tokens, residuals=None):
    """logits [T, vocab] of one sequence; residuals (a list) receives the stream after every layer."""
    eps = config["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    cached = {}
    for i, layer in enumerate(config["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        h = dyt(x, W, p + "norm1")
        if "kv_from" in mx:
            rows = cached[mx["kv_from"]]
        else:
            rows = cached[i] = latent_rows(h, W, p + "mix.", mx, eps)
        x = x + W[p + "ls1"] * dyt(mixer_latent(h, W, p + "mix.", mx, eps, rows), W, p + "norm1b")
        ml = layer["mlp"]
        if ml is not None:
            h = dyt(x, W, p + "norm2")
            y = feed_forward_dense(h, W, p + "mlp.") if ml["kind"] == "dense" else feed_forward_moe(h, W, p + "mlp.", ml)
            x = x + W[p + "ls2"] * dyt(y, W, p + "norm2b")
        if residuals is not None:
            residuals.append(x.clone())
    logits = dyt(x, W, "final.norm") @ W["head"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(config, W, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(forward(config, W, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


# ------------------------------------------------------------------ small random models
def latent_layer(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=32, window=24, scale=0.25, base=1000.0, rot_dims=None, kv_from=None, mlp=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "mask": {"size": window},
          "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=2, top=2, ff=24, shared_ff=40):
    ml = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared_ff:
        ml["shared"] = {"ff": shared_ff}
    return ml


def make_config(layers, width=48, vocab=61, eps=1e-5, embed_scale=3.0, softcap=12.0):
    return {"architecture": "Zefenex", "embedding": {"scale": embed_scale}, "layers": layers, "logit_softcap": softcap, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def make_weights(config, seed=0):
    """Random tensors with the checkpoint's names, every value exactly representable in bfloat16 (so that a bf16 engine, an fp32 engine and
    this float64 oracle all hold the same model).  Returns (float64 dict for the oracle, bf16 dict for the package)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = config["width"], config["vocab"]
    t = {}

    def mat(name, out, inn, gain=1.0):
        t[name] = torch.randn(out, inn, generator=g) * (gain / math.sqrt(inn))

    def vec(name, n, mean=1.0, spread=0.2):
        t[name] = mean + spread * torch.randn(n, generator=g)

    def norm(name):
        vec(name, width), vec(name + ".b", width, 0.0, 0.1)
        t[name + ".alpha"] = (0.6 + 0.3 * torch.rand((), generator=g))

    t["embed"] = 0.4 * torch.randn(vocab, width, generator=g)
    for i, layer in enumerate(config["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        H, d, dr, dv, r = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
        norm(p + "norm1"), norm(p + "norm1b"), vec(p + "ls1", width, 0.8, 0.2)
        mat(p + "mix.q", H * (d + dr), width, 2.0), mat(p + "mix.g", H * dv, width), mat(p + "mix.o", width, H * dv)
        mat(p + "mix.uk", H * d, r, 2.0), mat(p + "mix.uv", H * dv, r), vec(p + "mix.sink", H, 0.5, 1.0)
        if "kv_from" not in mx:
            mat(p + "mix.dkv", r + dr, width, 2.0), vec(p + "mix.dkv.norm", r, 1.2, 0.3)
        ml = layer["mlp"]
        if ml is None:
            continue
        norm(p + "norm2"), norm(p + "norm2b"), vec(p + "ls2", width, 0.8, 0.2)
        if ml["kind"] == "dense":
            mat(p + "mlp.up", ml["ff"], width), vec(p + "mlp.up.b", ml["ff"], 0.1, 0.3), mat(p + "mlp.down", width, ml["ff"])
            vec(p + "mlp.down.b", width, 0.0, 0.3)
            continue
        n_out = ml["router"]["experts"] + ml["router"].get("identity", 0)
        mat(p + "mlp.router", n_out, width, 3.0), vec(p + "mlp.correction", n_out, 0.0, 0.05)
        for e in range(ml["router"]["experts"]):
            mat(f"{p}mlp.e{e}.gate", ml["expert"]["ff"], width), mat(f"{p}mlp.e{e}.up", ml["expert"]["ff"], width)
            mat(f"{p}mlp.e{e}.down", width, ml["expert"]["ff"])
        if ml.get("shared"):
            f = ml["shared"]["ff"]
            mat(p + "mlp.shared.gate", f, width), mat(p + "mlp.shared.up", f, width), mat(p + "mlp.shared.down", width, f)
    norm("final.norm")
    mat("head", vocab, width, 3.0)
    packed = {k: v.to(torch.bfloat16) for k, v in t.items()}
    return {k: v.to(F) for k, v in packed.items()}, packed


def rel_err(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
