"""Zefenex: a decoder-only design of latent-attention layers --

  * mixer "latent_attention": the keys and values of all heads are up-projections (W_uk, W_uv) of one low-rank row c per position (the
    RMS-normed first kv_rank outputs of W_dkv), plus one rotated key part of rot_dim dimensions shared by the heads (the last rot_dim
    outputs of W_dkv); a query head is [dim un-rotated | rot_dim rotated]; rotation in the rotate-half layout over the first rot.dims of
    the rotated part; sliding window (i sees j with 0 <= i - j < mask.size); a learned per-head sink logit in the softmax denominator; a
    sigmoid output gate read from the mixer's input.  Only c and the rotated key part are cached.  A layer with "kv_from": j projects no
    rows of its own and reads layer j's cached rows through its own W_uk / W_uv;
  * feed-forward "dense": W_down relu(W_up h + b)^2 + b;  "moe": softmax router over experts + identity experts, choice by score +
    correction, weights = chosen scores / their sum, gated silu experts, identity experts return their input, an always-on shared expert;
  * every sublayer between two Dynamic-Tanh norms (tanh(alpha x) * w + b), its result scaled per channel (ls1 / ls2);
  * scaled embedding, Dynamic-Tanh final norm, soft-capped logits.

config.json gives every size; this module turns it plus the checkpoint's tensors into the layer list of hybrid.HybridDecoder: projections
that read the same input are fused into one matrix (q | gate | dkv), W_uk is stored per head transposed (the engine moves the query into
the latent space instead of the keys out of it), gate and up rows of an expert are stacked, the experts' matrices are stacked, each norm's
(w, b, alpha) becomes one fp32 vector."""
import importlib
import os

from . import register


def _pkg(sub=None):
    base = __package__.rsplit(".", 1)[0]
    return importlib.import_module(base + ("." + sub if sub else ""))


def layer_specs(config):
    """The integer / float side of every layer, straight from config.json (no tensors yet)."""
    m = _pkg()
    out = []
    for i, layer in enumerate(config["layers"]):
        mx, kind = layer["mixer"], layer["type"]
        if kind != "latent_attention":
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        rot = mx.get("rot") or {}
        rot_dim = int(mx.get("rot_dim", 0))
        spec = dict(mixer=m.MIXER_LATENT, norm=m.NORM_DYT_PRE_POST, heads=int(mx["heads"]), kv_heads=1, dim=int(mx["dim"]), vdim=int(mx["vdim"]),
                    kv_rank=int(mx["kv_rank"]), rot_dim=rot_dim, rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)),
                    scale=float(mx["scale"]), window=int((mx.get("mask") or {}).get("size", 0)), kv_from=int(mx.get("kv_from", -1)))
        if spec["kv_from"] >= i:
            raise ValueError(f"layer {i}: kv_from {spec['kv_from']} is not an earlier layer")
        mlp = layer.get("mlp")
        if mlp is None:
            spec.update(mlp=m.MLP_NONE)
        elif mlp["kind"] == "dense":
            spec.update(mlp=m.MLP_DENSE, expert_ff=int(mlp["ff"]), act=m.ACT_RELU2, gated=0)
        elif mlp["kind"] == "moe":
            shared, router = mlp.get("shared"), mlp["router"]
            spec.update(mlp=m.MLP_MOE, route=m.ROUTE_SOFTMAX, experts=int(router["experts"]), identity=int(router.get("identity", 0)),
                        top=int(router["top"]), expert_ff=int(mlp["expert"]["ff"]), shared_ff=int(shared["ff"]) if shared else 0, act=m.ACT_SILU,
                        gated=1)
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        out.append(spec)
    return out


def pack_norm(get, name, device):
    """(w, b, alpha) of one Dynamic-Tanh norm as the fp32 vector [w | b | alpha] the engine reads."""
    import torch

    return torch.cat([get(name).float().reshape(-1), get(name + ".b").float().reshape(-1), get(name + ".alpha").float().reshape(1)]).to(device).contiguous()


def fuse_layer(spec, get, width, dtype, device):
    """Adds the device tensors of one layer to its spec.  get(name) -> CPU tensor of the checkpoint ('mix.q', 'mlp.e0.up', ...)."""
    import torch

    m = _pkg()

    def mat(*names):
        ts = [get(n) for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).to(device=device, dtype=dtype).contiguous()

    def vec(name):
        return get(name).to(device=device, dtype=torch.float32).reshape(-1).contiguous()

    H, dim, vdim, rank = spec["heads"], spec["dim"], spec["vdim"], spec["kv_rank"]
    own = spec["kv_from"] < 0
    spec.update(w_in=mat("mix.q", "mix.g", "mix.dkv") if own else mat("mix.q", "mix.g"), w_out=mat("mix.o"), sink=vec("mix.sink"),
                w_uk_t=get("mix.uk").reshape(H, dim, rank).transpose(1, 2).to(device=device, dtype=dtype).contiguous(),
                w_uv=get("mix.uv").reshape(H, vdim, rank).to(device=device, dtype=dtype).contiguous(),
                pre1=pack_norm(get, "norm1", device), post1=pack_norm(get, "norm1b", device), ls1=vec("ls1"))
    if own:
        spec["kv_norm"] = vec("mix.dkv.norm")
    if spec["mlp"] == m.MLP_NONE:
        return spec
    spec.update(pre2=pack_norm(get, "norm2", device), post2=pack_norm(get, "norm2b", device), ls2=vec("ls2"))
    if spec["mlp"] == m.MLP_DENSE:
        spec.update(w_up=mat("mlp.up"), b_up=vec("mlp.up.b"), w_down=mat("mlp.down"), b_down=vec("mlp.down.b"))
    else:
        E = spec["experts"]
        spec.update(w_router=mat("mlp.router"), route_bias=vec("mlp.correction"),
                    w_up=torch.stack([torch.cat([get(f"mlp.e{e}.gate"), get(f"mlp.e{e}.up")], 0) for e in range(E)]).to(device=device, dtype=dtype).contiguous(),
                    w_down=torch.stack([get(f"mlp.e{e}.down") for e in range(E)]).to(device=device, dtype=dtype).contiguous())
        if spec["shared_ff"]:
            spec.update(w_shared_up=mat("mlp.shared.gate", "mlp.shared.up"), w_shared_down=mat("mlp.shared.down"))
    return spec


@register("Zefenex")
class ZefenexModel:
    """config + tensors -> a HybridDecoder.  `tensors`: name -> CPU tensor with the checkpoint's names ('embed', 'l0.mix.q', ..., 'head')."""

    def __init__(self, config, tensors, dtype="bfloat16", device="cuda:0", max_tokens=2048, max_seqs=4, max_pages_per_seq=None):
        import torch

        m = _pkg()
        tdt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[dtype] if isinstance(dtype, str) else dtype
        self.config, self.width, self.vocab = config, int(config["width"]), int(config["vocab"])
        self.eps = float(config["norm"]["eps"])
        specs = layer_specs(config)
        for i, spec in enumerate(specs):
            fuse_layer(spec, lambda n, i=i: tensors[f"l{i}.{n}"], self.width, tdt, device)
        if max_pages_per_seq is None:
            max_pages_per_seq = (max_tokens + m.KV_PAGE_SIZE - 1) // m.KV_PAGE_SIZE
        self.engine = _pkg("hybrid").HybridDecoder(
            self.width, self.vocab, self.eps, specs, tensors["embed"].to(device=device, dtype=tdt).contiguous(),
            pack_norm(lambda n: tensors[n], "final.norm", device), tensors["head"].to(device=device, dtype=tdt).contiguous(),
            tdt, device, max_tokens, max_seqs, max_pages_per_seq, embed_scale=float((config.get("embedding") or {}).get("scale", 1.0)),
            logit_softcap=float(config.get("logit_softcap") or 0.0), final_norm_kind=m.NORM_DYT_PRE_POST)

    @classmethod
    def from_pretrained(cls, model_dir, config, dtype="bfloat16", device="cuda:0", **limits):
        tensors = _pkg("weights").read_safetensors(os.path.join(model_dir, "model.safetensors"))
        return cls(config, tensors, dtype=dtype, device=device, **limits)
