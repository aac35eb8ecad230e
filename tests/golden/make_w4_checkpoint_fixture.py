"""Regenerates tests/golden/tiny_w4_ckpt/ from the reference's own tools.

Run in a container that holds the reference tree (environment variable REF_ROOT points at it):
    python tests/golden/make_w4_checkpoint_fixture.py
It runs tools/make_tiny_checkpoint.py (fp32 checkpoint, seed 1234) and
tools/convert_hf_to_glmserve.py --quantize-int4 --group 16 (the W4 checkpoint) into a temporary
folder and keeps, byte for byte, only what the MLP half needs:

  config.json          the converter's output config
  model.safetensors    the `.mlp.` tensors of layer 0 (dense MLP) and layer 2 (first MoE layer) of
                       the W4 checkpoint, tensor bytes copied unchanged
  fp/fp_subset.safetensors  the fp32 originals of a few of those linears: the quantiser twin
                       (glmserve_b200.quant.quantize_w4_np) must reproduce the converter's
                       nibbles and scales from them
  expected.npz         x (bf16-representable) and out_ref = GLM52Model::moe_mlp (compiled from the
                       reference sources, oracle/_ref) on layer 2 as loaded by
                       glmserve_b200.checkpoint
The GPU box never runs this script; it only reads the files.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF_ROOT = os.environ.get("REF_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
if not os.path.isdir(os.path.join(REF_ROOT, "tools")):
    sys.exit("set REF_ROOT to the reference checkout (its tools/ folder is imported to generate the vectors)")

import oracle  # noqa: E402
from glmserve_b200.checkpoint import Checkpoint, SafetensorsFile, write_safetensors  # noqa: E402
from glmserve_b200.quant import round_bf16_np  # noqa: E402


def subset(src: SafetensorsFile, keep) -> dict:
    out = {}
    for name in src.names():
        if keep(name):
            t = src.tensor(name)
            out[name] = ("BF16", np.array(t)) if src.dtype(name) == "BF16" else np.array(t)
    return out


def main():
    oracle.build(with_ref=True)
    assert oracle.ref_available(), "reference tree not found; cannot regenerate the fixture"
    dst = os.path.join(HERE, "tiny_w4_ckpt")
    os.makedirs(dst, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        fp, w4 = os.path.join(tmp, "fp"), os.path.join(tmp, "w4")
        subprocess.run([sys.executable, os.path.join(REF_ROOT, "tools", "make_tiny_checkpoint.py"), "--out", fp],
                       check=True, capture_output=True)
        subprocess.run([sys.executable, os.path.join(REF_ROOT, "tools", "convert_hf_to_glmserve.py"), "--model", fp,
                        "--quantize-int4", w4, "--group", "16"], check=True, capture_output=True)
        shutil.copy(os.path.join(w4, "config.json"), os.path.join(dst, "config.json"))
        mlp = lambda n: n.startswith("model.layers.0.mlp.") or n.startswith("model.layers.2.mlp.")
        write_safetensors(os.path.join(dst, "model.safetensors"),
                          subset(SafetensorsFile(os.path.join(w4, "model.safetensors")), mlp))
        few = ("model.layers.2.mlp.experts.0.", "model.layers.2.mlp.experts.5.down_proj",
               "model.layers.2.mlp.shared_experts.", "model.layers.2.mlp.gate.", "model.layers.0.mlp.gate_proj")
        os.makedirs(os.path.join(dst, "fp"), exist_ok=True)   # apart: a checkpoint folder's shards are all read
        write_safetensors(os.path.join(dst, "fp", "fp_subset.safetensors"),
                          subset(SafetensorsFile(os.path.join(fp, "model.safetensors")),
                                 lambda n: any(n.startswith(p) for p in few)))
    ck = Checkpoint(dst)
    L = ck.load_moe_layer(2)
    rng = np.random.default_rng(2024)
    x = round_bf16_np(rng.standard_normal((24, L["H"])).astype(np.float32))
    out_ref, _ = oracle.ref_moe_mlp_w4(x, L)
    np.savez(os.path.join(dst, "expected.npz"), x=x, out_ref=out_ref)
    for base, _, files in os.walk(dst):
        for fn in sorted(files):
            print(os.path.relpath(os.path.join(base, fn), dst), os.path.getsize(os.path.join(base, fn)), "bytes")


if __name__ == "__main__":
    main()
