"""lb-convert on the GPU: `python -m lemonade_burn_b200.convert --src <hf model dir> --dst <out dir>
[--check <quant_summary.json>]`, the command line of crates/lb-convert/src/main.rs:19-28.

Reads the bf16 master weights (`model.safetensors`), ternarises every BitLinear weight as
`transformers`' WeightQuant does (lb-ternary/src/pack.rs:118-142), packs it four weights per byte
(pack.rs:88-103) and writes `model.lbt.safetensors` in the format of lb-convert/src/lib.rs:1-16. The
arithmetic (absmean with an f64 sum, ties-to-even ternarisation, packing, the counts and the sha256
of each ternary int8 array) runs in liblbk.so on the GPU (`lbk_convert_bitlinear`); torch is used
to hold device memory and safetensors to read and write the files. With `--check`, each tensor's
sha256 and scale are compared with the summary scripts/hf_reference.py writes (main.rs:141-170).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import shutil
import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from .pack import row_bytes
from .ternary import Context, default_context

FORMAT = "lemonade-burn-ternary"   # lb-convert/src/lib.rs:14-16
VERSION = "1"
FILE_NAME = "model.lbt.safetensors"
LINEAR_SUFFIXES = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                   "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")   # lib.rs:18-26
QUANT_NOTE = "weights: absmean per-tensor ternary (WeightQuant); acts: per-token absmax int8 at runtime"
LAYOUT_NOTE = "row-major, 128-weight blocks of 32 bytes, bits 2k..2k+1 of byte j = code(w+1) of weight k*32+j"


def is_bitlinear_weight(name: str) -> bool:
    """lib.rs:30-33."""
    return name.startswith("model.layers.") and any(name.endswith(s + ".weight") for s in LINEAR_SUFFIXES)


class _Item(C.Structure):
    _fields_ = [("src_dev", C.c_void_p), ("rows", C.c_size_t), ("cols", C.c_size_t), ("packed_dev", C.c_void_p)]


@dataclass
class Converted:
    packed: torch.Tensor            # uint8 [rows, row_bytes(cols)] on the GPU: `<linear>.qweight`
    scale: np.float32               # `<linear>.wscale` = 1 / mean|W|
    counts: Tuple[int, int, int]    # how many -1, 0, +1
    sha256: Optional[str]           # of the int8 ternary array [rows*cols], hex


def convert_bitlinear(weights: Sequence[torch.Tensor], ctx: Optional[Context] = None, sha: bool = True) -> List[Converted]:
    """main.rs:62-87 for a list of rank-2 CUDA tensors, all bf16 or all f32."""
    if not weights:
        return []
    ctx = ctx or default_context()
    dt = weights[0].dtype
    if dt not in (torch.bfloat16, torch.float32):
        raise TypeError("master weights must be bf16 or f32")
    ws = []
    for w in weights:
        if w.dtype != dt:
            raise TypeError("all tensors of one call must share a dtype")
        if w.dim() != 2 or not w.is_cuda:
            raise ValueError("expected rank-2 CUDA tensors")
        ws.append(w.contiguous())
    n = len(ws)
    packed = [torch.empty((w.shape[0], row_bytes(w.shape[1])), dtype=torch.uint8, device=w.device) for w in ws]
    items = (_Item * n)(*[_Item(w.data_ptr(), w.shape[0], w.shape[1], p.data_ptr()) for w, p in zip(ws, packed)])
    scales = np.empty(n, dtype=np.float32)
    counts = np.empty((n, 3), dtype=np.uint64)
    digests = np.empty((n, 32), dtype=np.uint8) if sha else None
    _lib.check(ctx._lib.lbk_convert_bitlinear(ctx.handle, C.cast(items, C.c_void_p), n, 1 if dt == torch.bfloat16 else 0,
                                              scales.ctypes.data_as(C.c_void_p), counts.ctypes.data_as(C.c_void_p),
                                              digests.ctypes.data_as(C.c_void_p) if sha else None,
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return [Converted(packed[i], scales[i], tuple(int(c) for c in counts[i]), digests[i].tobytes().hex() if sha else None)
            for i in range(n)]


def convert_checkpoint(src, dst, check=None, ctx: Optional[Context] = None, device: str = "cuda", log=sys.stderr) -> Dict[str, dict]:
    """The converter's main (main.rs:43-171). Returns {tensor name: {scale, sha256, counts}} for the
    BitLinear weights; raises ValueError on an unexpected tensor or dtype (main.rs:58-60,105),
    SystemExit(2) when --check finds different ternary values (main.rs:166-168)."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    src, dst = Path(src), Path(dst)
    t0 = time.perf_counter()
    outs: Dict[str, torch.Tensor] = {}
    lin_names: List[str] = []
    lin_w: List[torch.Tensor] = []
    with safe_open(str(src / "model.safetensors"), "pt", device=device) as f:
        for name in sorted(f.keys()):
            t = f.get_tensor(name)
            if t.dtype != torch.bfloat16:
                raise ValueError(f"{name}: expected BF16, got {t.dtype}")
            if is_bitlinear_weight(name):
                lin_names.append(name)
                lin_w.append(t)
            elif name.endswith("norm.weight"):
                outs[name] = t.float()            # bf16 widened, exact
            elif name == "model.embed_tokens.weight":
                outs[name] = t
            else:
                raise ValueError(f"unexpected tensor {name}")
    conv = convert_bitlinear(lin_w, ctx)
    qinfo: Dict[str, dict] = {}
    for name, c in zip(lin_names, conv):
        linear = name[: -len(".weight")]
        outs[linear + ".qweight"] = c.packed
        outs[linear + ".wscale"] = torch.tensor([c.scale], dtype=torch.float32)
        qinfo[name] = {"scale": float(c.scale), "sha256": c.sha256, "counts": {"-1": c.counts[0], "0": c.counts[1], "1": c.counts[2]}}
    print(f"ternarized {len(conv)} BitLinear tensors in {time.perf_counter() - t0:.1f}s", file=log)
    dst.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous().cpu() for k, v in outs.items()}, str(dst / FILE_NAME),
              metadata={"format": FORMAT, "version": VERSION, "quant": QUANT_NOTE, "layout": LAYOUT_NOTE})
    for fn in ("config.json", "tokenizer.json", "tokenizer_config.json", "generation_config.json", "LICENSE"):
        if (src / fn).exists():
            shutil.copy(src / fn, dst / fn)
    size = (dst / FILE_NAME).stat().st_size
    print(f"wrote {dst / FILE_NAME} ({size / 1e6:.1f} MB) in {time.perf_counter() - t0:.1f}s", file=log)
    tot = [sum(q["counts"][k] for q in qinfo.values()) for k in ("-1", "0", "1")]
    nw = max(sum(tot), 1)
    print(f"ternary distribution: -1 {100 * tot[0] / nw:.2f}%  0 {100 * tot[1] / nw:.2f}%  +1 {100 * tot[2] / nw:.2f}%  ({nw} weights)", file=log)
    if check is not None:
        summary = json.loads(Path(check).read_text())
        ok = bad_sha = bad_scale = 0
        for name, q in qinfo.items():
            s = summary.get(name)
            if s is None:
                raise ValueError(f"{name} missing from {check}")
            scale_ok = np.float32(s["scale"]).tobytes() == np.float32(q["scale"]).tobytes()
            sha_ok = s["sha256"] == q["sha256"]
            if not scale_ok:
                bad_scale += 1
                print(f"  scale mismatch {name}: ours {q['scale']:e} torch {s['scale']:e}", file=log)
            if not sha_ok:
                bad_sha += 1
                print(f"  ternary mismatch {name}", file=log)
            ok += scale_ok and sha_ok
        print(f"check vs torch: {ok}/{len(qinfo)} identical, {bad_scale} scale mismatches, {bad_sha} ternary mismatches", file=log)
        if bad_sha:
            raise SystemExit(2)
    return qinfo


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--check", default=None, help="quant_summary.json from scripts/hf_reference.py")
    a = ap.parse_args(argv)
    convert_checkpoint(a.src, a.dst, a.check)
    return 0


if __name__ == "__main__":
    sys.exit(main())
