"""Llama-2 family on the fused decoder engine (a checkpoint packed by weights.save_packed; see scripts/convert_weights.py)."""
import importlib

from . import register


def _weights():
    return importlib.import_module(__package__.rsplit(".", 1)[0] + ".weights")


@register("Llama", "LlamaForCausalLM", "llama")
class LlamaModel:
    def __init__(self, decoder, packed, shape):
        self.decoder, self.packed, self.shape = decoder, packed, shape

    @classmethod
    def from_pretrained(cls, model_dir, config, dtype="bfloat16", device="cuda:0", max_seq=2048, max_batch=1, **_):
        w = _weights()
        packed, manifest = w.load_packed(model_dir, device)
        shape = manifest["shape"]
        dec, packed = w.build_decoder(packed, shape, device, manifest["dtype"], manifest["wformat"], max_seq, max_batch,
                                      group=manifest.get("group", 128))
        return cls(dec, packed, shape)
