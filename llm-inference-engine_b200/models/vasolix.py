"""Vasolix: a decoder-only design whose layers alternate freely between two token mixers --

  * "attention": softmax attention with no rotation; keys double as values (v = k as projected, before the key norm); q and k are RMS-normed
    over their WHOLE projection (all heads at once); grouped key/value heads; a block-diagonal causal mask (position i sees j <= i in the
    same block of mask.size positions, blocks counted from position 0); a learned per-head sink logit in the softmax denominator; a
    sigmoid output gate read from the mixer's input;
  * "gla": gated linear attention, S <- diag(a) S + k v^T, o = S^T q / sqrt(dim), with a = sigmoid(W2 W1 h + b)^(1/tau) per key channel,
    per-head RMS norm of o with one shared weight, a silu output gate --

each followed by a mixture-of-experts feed-forward (sigmoid router, top-k scores used un-normalised as weights ON THE EXPERT'S INPUT,
squared-relu experts, a sigmoid-gated shared expert), with the RMS norm on every sublayer's OUTPUT and an fp32 residual stream.

config.json gives every size; this module turns it plus the checkpoint's tensors into the layer list of hybrid.HybridDecoder:
projections that read the same input are fused into one matrix (attention: q | k | gate; gla: q | k | v | gate | decay-in), the experts'
matrices are stacked, small vectors become fp32."""
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
        spec = dict(heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])))
        if kind == "attention":
            mask = mx.get("mask") or {}
            spec.update(mixer=m.MIXER_ATTN_CHUNKED, kv_heads=int(mx.get("kv_heads", mx["heads"])), scale=float(mx["scale"]),
                        chunk=int(mask.get("size", 0)))
        elif kind == "gla":
            spec.update(mixer=m.MIXER_GLA, kv_heads=int(mx["heads"]), tau=float(mx["tau"]))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = layer.get("mlp")
        if mlp is None:
            spec.update(mlp=m.MLP_NONE)
        elif mlp.get("kind", "moe") == "moe":
            shared = mlp.get("shared")
            spec.update(mlp=m.MLP_MOE, experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]), expert_ff=int(mlp["expert"]["ff"]),
                        shared_ff=int(shared["ff"]) if shared else 0, act=m.ACT_RELU2)
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        out.append(spec)
    return out


def fuse_layer(spec, get, width, dtype, device):
    """Adds the device tensors of one layer to its spec.  get(name) -> CPU tensor of the checkpoint ('mix.q', 'mlp.e0.up', ...)."""
    import torch

    m = _pkg()

    def mat(*names):
        ts = [get(n) for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).to(device=device, dtype=dtype).contiguous()

    def vec(name):
        return get(name).to(device=device, dtype=torch.float32).reshape(-1).contiguous()

    if spec["mixer"] == m.MIXER_ATTN_CHUNKED:
        spec.update(w_in=mat("mix.q", "mix.k", "mix.g"), w_out=mat("mix.o"), q_norm=vec("mix.q.norm"), k_norm=vec("mix.k.norm"),
                    sink=vec("mix.sink"))
    else:
        spec.update(w_in=mat("mix.q", "mix.k", "mix.v", "mix.g", "mix.a1"), w_out=mat("mix.o"), w_decay=mat("mix.a2"),
                    decay_bias=vec("mix.a2.b"), out_norm=vec("mix.norm"), decay_rank=int(get("mix.a1").shape[0]))
    spec["norm1"] = vec("norm1")
    if spec["mlp"] == m.MLP_MOE:
        E = spec["experts"]
        gate_row = get("mlp.shared.sg").reshape(1, width) if spec["shared_ff"] else torch.zeros(1, width)
        spec.update(norm2=vec("norm2"),
                    w_router=torch.cat([get("mlp.router").float(), gate_row.float()], 0).to(device=device, dtype=dtype).contiguous(),
                    w_up=torch.stack([get(f"mlp.e{e}.up") for e in range(E)]).to(device=device, dtype=dtype).contiguous(),
                    w_down=torch.stack([get(f"mlp.e{e}.down") for e in range(E)]).to(device=device, dtype=dtype).contiguous())
        if spec["shared_ff"]:
            spec.update(w_shared_up=mat("mlp.shared.up"), w_shared_down=mat("mlp.shared.down"))
    return spec


@register("Vasolix")
class VasolixModel:
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
            tensors["final.norm"].to(device=device, dtype=torch.float32).contiguous(), tensors["head"].to(device=device, dtype=tdt).contiguous(),
            tdt, device, max_tokens, max_seqs, max_pages_per_seq)

    @classmethod
    def from_pretrained(cls, model_dir, config, dtype="bfloat16", device="cuda:0", **limits):
        tensors = _pkg("weights").read_safetensors(os.path.join(model_dir, "model.safetensors"))
        return cls(config, tensors, dtype=dtype, device=device, **limits)
