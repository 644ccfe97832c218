"""Plain, slow restatement of the Vasolix design in float64 on the CPU, one function per mechanism, written from the design's
equations and sharing nothing with the package: the oracle for tests/test_vasolix*.py.

Notation: h is a [T, width] block of one sequence's tokens at positions 0..T-1; W['name'] are float64 matrices stored [out, in].
Every function sees the WHOLE sequence at once (no cache, no state carried between calls): whatever the engine does with pages, slots,
portions and batches must reproduce these numbers."""
import math

import numpy as np
import torch

F = torch.float64


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def mixer_attention(h, W, p, mx, eps):
    """softmax(scale q.k + block-diagonal causal mask, plus one sink logit per head) applied to v = un-normed k; sigmoid gate."""
    T = h.shape[0]
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    q_raw, k_raw = h @ W[p + "q"].T, h @ W[p + "k"].T
    q = (rms_unit(q_raw, eps) * W[p + "q.norm"]).view(T, H, d)      # one norm over all heads' channels together
    k = (rms_unit(k_raw, eps) * W[p + "k.norm"]).view(T, G, d)
    v = k_raw.view(T, G, d)
    size = mx["mask"]["size"]
    i = torch.arange(T)
    visible = (i[None, :] <= i[:, None]) & (torch.div(i[None, :], size, rounding_mode="floor") == torch.div(i[:, None], size, rounding_mode="floor"))
    heads = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * mx["scale"]
        e = torch.where(visible, torch.exp(s), torch.zeros_like(s))
        denom = e.sum(-1, keepdim=True) + torch.exp(W[p + "sink"][a])
        heads.append((e / denom) @ v[:, g])
    o = torch.cat(heads, -1) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def gla_decay(h, W, p, mx):
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    return torch.sigmoid(z) ** (1.0 / mx["tau"])


def mixer_gla(h, W, p, mx, eps):
    T = h.shape[0]
    H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, d) / math.sqrt(d)
    k = (h @ W[p + "k"].T).view(T, H, d)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    a = gla_decay(h, W, p, mx).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = a[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = (S * q[t].unsqueeze(-1)).sum(1)
    o = (rms_unit(o, eps) * W[p + "norm"]).reshape(T, H * dv)
    gate = h @ W[p + "g"].T
    return (o * gate * torch.sigmoid(gate)) @ W[p + "o"].T


def relu2_expert(x, W, p):
    return (torch.relu(x @ W[p + "up"].T) ** 2) @ W[p + "down"].T


def route(h, W, p, ml):
    score = torch.sigmoid(h @ W[p + "router"].T)
    weight, chosen = torch.topk(score, ml["router"]["top"], dim=-1)
    return chosen, weight


def feed_forward_moe(h, W, p, ml):
    chosen, weight = route(h, W, p, ml)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weight[t]):
            y[t] += relu2_expert(w * h[t], W, f"{p}e{e}.")   # the weight scales the expert's input
    if ml.get("shared"):
        y = y + relu2_expert(h, W, p + "shared.") * torch.sigmoid(h @ W[p + "shared.sg"].T)
    return y


def forward(config, W, tokens, residuals=None):
    """logits [T, vocab] of one sequence; residuals (a list) receives the stream after every layer."""
    eps = config["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mix = {"attention": mixer_attention, "gla": mixer_gla}[layer["type"]]
        x = x + rms_unit(mix(x, W, p + "mix.", layer["mixer"], eps), eps) * W[p + "norm1"]
        if layer["mlp"] is not None:
            x = x + rms_unit(feed_forward_moe(x, W, p + "mlp.", layer["mlp"]), eps) * W[p + "norm2"]
        if residuals is not None:
            residuals.append(x.clone())
    return (rms_unit(x, eps) * W["final.norm"]) @ W["head"].T


def greedy(config, W, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(forward(config, W, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


# ------------------------------------------------------------------ small random models
def attention_layer(heads=4, kv_heads=2, dim=16, size=24, scale=0.3, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": size}}, "mlp": mlp}


def gla_layer(heads=2, dim=16, vdim=24, tau=7.0, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def moe(experts=5, top=2, ff=24, shared_ff=40):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": shared_ff}}


def make_config(layers, width=48, vocab=61, eps=1e-5):
    return {"architecture": "Vasolix", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def make_weights(config, seed=0, decay_rank=6):
    """Random tensors with the checkpoint's names, every value exactly representable in bfloat16 (so that a bf16 engine, an fp32 engine and
    this float64 oracle all hold the same model).  Returns (float64 dict for the oracle, bf16 dict for the package)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = config["width"], config["vocab"]
    t = {}

    def mat(name, out, inn, gain=1.0):
        t[name] = torch.randn(out, inn, generator=g) * (gain / math.sqrt(inn))

    def vec(name, n, mean=1.0, spread=0.2):
        t[name] = mean + spread * torch.randn(n, generator=g)

    t["embed"] = torch.randn(vocab, width, generator=g)
    for i, layer in enumerate(config["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        H, d = mx["heads"], mx["dim"]
        vec(p + "norm1", width)
        if layer["type"] == "attention":
            G = mx["kv_heads"]
            mat(p + "mix.q", H * d, width), mat(p + "mix.k", G * d, width), mat(p + "mix.g", H * d, width), mat(p + "mix.o", width, H * d)
            vec(p + "mix.q.norm", H * d, 1.5, 0.4), vec(p + "mix.k.norm", G * d, 1.5, 0.4), vec(p + "mix.sink", H, 0.5, 1.0)
        else:
            dv = mx["vdim"]
            mat(p + "mix.q", H * d, width), mat(p + "mix.k", H * d, width), mat(p + "mix.v", H * dv, width), mat(p + "mix.g", H * dv, width)
            mat(p + "mix.o", width, H * dv), mat(p + "mix.a1", decay_rank, width), mat(p + "mix.a2", H * d, decay_rank, 2.0)
            vec(p + "mix.a2.b", H * d, 1.0, 1.5), vec(p + "mix.norm", dv)
        ml = layer["mlp"]
        if ml is not None:
            vec(p + "norm2", width)
            mat(p + "mlp.router", ml["router"]["experts"], width, 2.0)
            for e in range(ml["router"]["experts"]):
                mat(f"{p}mlp.e{e}.up", ml["expert"]["ff"], width), mat(f"{p}mlp.e{e}.down", width, ml["expert"]["ff"])
            if ml.get("shared"):
                mat(p + "mlp.shared.up", ml["shared"]["ff"], width), mat(p + "mlp.shared.down", width, ml["shared"]["ff"])
                mat(p + "mlp.shared.sg", 1, width, 2.0)
    vec("final.norm", width)
    mat("head", vocab, width)
    packed = {k: v.to(torch.bfloat16) for k, v in t.items()}
    return {k: v.to(F) for k, v in packed.items()}, packed


def rel_err(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
