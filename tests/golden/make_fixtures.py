"""Generates tests/golden/hf_bitnet_quant.npz from the installed `transformers` BitNet
integration (ActQuant / WeightQuant), which the reference states it reproduces
(crates/lb-ternary/src/quant.rs:1-10, crates/lb-ternary/src/pack.rs:118-128) and validates
against (scripts/hf_reference.py:41-58).

Run once where transformers + torch are installed:  python tests/golden/make_fixtures.py
The library functions are decorated with torch.compile; TORCHDYNAMO_DISABLE=1 makes them
run eagerly, which is the arithmetic being pinned. Inputs are seeded and stored next to the
library's outputs, so the tests need neither torch nor transformers.
"""
import os

os.environ["TORCHDYNAMO_DISABLE"] = "1"

from pathlib import Path

import numpy as np
import torch
from transformers.integrations.bitnet import ActQuant, WeightQuant

OUT = Path(__file__).resolve().parent / "hf_bitnet_quant.npz"


def main():
    g = torch.Generator().manual_seed(20251)
    fx = {}
    # activations: rows with outliers, an exact-tie row (amax 127 -> scale 1, values k+0.5),
    # a zero row and a tiny row
    x = torch.randn(6, 300, generator=g)
    x[0, 3] = 20.0
    x[1, ::97] *= 15.0
    ties = torch.arange(-48, 48, dtype=torch.float32) + 0.5
    x[2] = 0
    x[2, :96] = ties
    x[2, 96] = 127.0
    x[3] = 0.0
    x[4] = 1e-30
    fx["act_x"] = x.numpy().copy()
    fx["act_dequant"] = ActQuant.apply(x.clone()).numpy().copy()  # q / scale, f32
    # the library's own expressions, kept separately: scale and integer codes
    amax = x.abs().max(dim=-1, keepdim=True).values.clamp_(min=1e-5)
    scale = 127 / amax  # torch evaluates scalar / tensor as tensor.reciprocal() * scalar
    fx["act_scale"] = scale.reshape(-1).numpy().copy()
    fx["act_q"] = (x * scale).round().clamp(-128, 127).to(torch.int8).numpy().copy()

    # weights: three tensors with different spreads
    for i, (shape, std) in enumerate([((48, 300), 0.02), ((17, 128), 1.0), ((5, 1000), 3e-4)]):
        w = torch.randn(*shape, generator=g) * std
        fx[f"w{i}"] = w.numpy().copy()
        fx[f"w{i}_dequant"] = WeightQuant.apply(w.clone()).numpy().copy()  # t / scale
        fx[f"w{i}_scale"] = np.float32((1.0 / w.abs().mean().clamp_(min=1e-5)).item())
    np.savez_compressed(OUT, **fx)
    print("wrote", OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
