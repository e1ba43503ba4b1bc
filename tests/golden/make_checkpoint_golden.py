"""Generate ``tests/golden/packed_checkpoint_v1`` with the REFERENCE's own exporter.

Run in the build container (the reference tree is needed, at ``--reference``):

    python tests/golden/make_checkpoint_golden.py --reference /path/to/dynquant

A one-layer Llama-shaped model (hidden 128, intermediate 256, vocabulary 128, fp16, seeded) is
exported by ``dynquant.quant.checkpoint.export_packed_checkpoint`` with a different width on
the shards of every fused layer, an 8-bit lm_head and the embedding left dense.  Beside the
checkpoint the script stores what the reference decodes each packed module to
(``expected_dequant.npz``: fp16 bit patterns from ``QuantTensor.dequantize``), so that the
loader test can check values and not only keys.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference project")
    ns = ap.parse_args()
    sys.path.insert(0, str(Path(ns.reference) / "packages" / "dynquant-core" / "src"))
    import transformers
    from dynquant.quant.checkpoint import export_packed_checkpoint
    from dynquant.quant.device import quantize_tensor

    config = transformers.LlamaConfig(
        vocab_size=128, hidden_size=128, intermediate_size=256, num_hidden_layers=1,
        num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
        tie_word_embeddings=False,
    )
    torch.manual_seed(20260)
    model = transformers.LlamaForCausalLM(config).to(torch.float16).eval()
    widths = {"q_proj": 4, "k_proj": 2, "v_proj": 3, "o_proj": 8, "gate_proj": 3, "up_proj": 4, "down_proj": 2}
    bits = {}
    for name, module in model.named_modules():
        if isinstance(module, torch.nn.Linear):
            bits[name] = widths.get(name.rsplit(".", 1)[-1], 8)
    out = HERE / "packed_checkpoint_v1"
    report = export_packed_checkpoint(model, bits, output_dir=out, compute_device=None)
    expected = {}
    for name, width in sorted(bits.items()):
        module = model.get_submodule(name)
        qt, _ = quantize_tensor(module.weight.detach(), bits=width, group_size=128, symmetric=False,
                                compute_dtype=torch.float16, device=torch.device("cpu"))
        expected[name] = qt.dequantize().to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(out / "expected_dequant.npz", **expected)
    for extra in ("generation_config.json",):
        (out / extra).unlink(missing_ok=True)
    print(report.summary())
    print(sorted(p.name for p in out.iterdir()))


if __name__ == "__main__":
    main()
