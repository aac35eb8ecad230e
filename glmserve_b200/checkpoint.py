"""On-disk W4 checkpoint -> resident layer tensors -> tile streams.

Reads the format the reference's converter writes (tools/convert_hf_to_glmserve.py:216-251,
:323-380): a safetensors container in which every quantised linear ``X.weight [out, in]`` has
become ``X.qweight`` (U8 ``[out, in/2]``, two nibbles per byte, low nibble = even column, stored
value = q + 8) and ``X.scales`` (F32 ``[out, in/group]``).  Per-expert tensors are named
``model.layers.{i}.mlp.experts.{e}.{gate,up,down}_proj`` (docs/glm52_tensor_map.md:67-74,
src/model_glm52.cpp:279-296); this module gathers them into the ``[E, rows, cols/2]`` arrays
the engine concatenates at upload (src/model_gpu.cpp:948-1000) and that ``ops.MoELayer`` /
``gsb_prepack_*`` take.

The safetensors reader is self-contained (8-byte little-endian header length, JSON header,
raw little-endian tensor bytes) and memory-maps the file: nothing is copied until a tensor is
gathered.  ``python -m glmserve_b200.checkpoint DIR --layer 3 --out layer3.npz`` writes the
gathered arrays plus, where the shapes allow, the prepacked tile streams (numpy twin of the GPU
prepack, so it runs without a GPU).
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

_DTYPES = {"U8": np.uint8, "I8": np.int8, "F32": np.float32, "F16": np.float16, "BF16": np.uint16,
           "I32": np.int32, "I64": np.int64, "F64": np.float64, "BOOL": np.bool_}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            self.header = json.loads(f.read(hlen).decode("utf-8"))
        self.data_offset = 8 + hlen
        self.header.pop("__metadata__", None)
        self._mm = np.memmap(path, dtype=np.uint8, mode="r")

    def names(self):
        return list(self.header.keys())

    def has(self, name: str) -> bool:
        return name in self.header

    def dtype(self, name: str) -> str:
        return self.header[name]["dtype"]

    def tensor(self, name: str) -> np.ndarray:
        """A read-only view of the tensor's bytes (BF16 comes back as uint16 bit patterns)."""
        meta = self.header[name]
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"{name}: dtype {meta['dtype']} not supported by this reader")
        b, e = meta["data_offsets"]
        raw = self._mm[self.data_offset + b:self.data_offset + e]
        return raw.view(_DTYPES[meta["dtype"]]).reshape(meta["shape"])


def write_safetensors(path: str, tensors: dict) -> None:
    """Minimal writer (tests and fixtures): tensors in insertion order, header padded to 8 bytes."""
    rev = {np.dtype(v): k for k, v in _DTYPES.items() if k != "BF16"}
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        bf16 = isinstance(arr, tuple)          # ("BF16", uint16 array)
        a = np.ascontiguousarray(arr[1] if bf16 else arr)
        dt = "BF16" if bf16 else rev[a.dtype]
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        blobs.append(a.tobytes())
        off += a.nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class Checkpoint:
    """A directory holding ``config.json`` and one or more ``*.safetensors`` shards
    (``model.safetensors.index.json`` maps names to shards when there are several)."""

    def __init__(self, directory: str):
        self.dir = directory
        with open(os.path.join(directory, "config.json"), "r", encoding="utf-8") as f:
            self.config = json.load(f)
        self._files = {}
        idx = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx, "r", encoding="utf-8") as f:
                self.weight_map = dict(json.load(f)["weight_map"])
        else:
            self.weight_map = {}
            for fn in sorted(os.listdir(directory)):
                if fn.endswith(".safetensors"):
                    for name in self._file(fn).names():
                        self.weight_map[name] = fn

    def _file(self, fn: str) -> SafetensorsFile:
        if fn not in self._files:
            self._files[fn] = SafetensorsFile(os.path.join(self.dir, fn))
        return self._files[fn]

    def has(self, name: str) -> bool:
        return name in self.weight_map

    def tensor(self, name: str) -> np.ndarray:
        return self._file(self.weight_map[name]).tensor(name)

    def dtype(self, name: str) -> str:
        return self._file(self.weight_map[name]).dtype(name)

    def float_tensor(self, name: str) -> np.ndarray:
        """F32 / F16 / BF16 tensor as float32."""
        t = self.tensor(name)
        if self.dtype(name) == "BF16":
            return (t.astype(np.uint32) << 16).view(np.float32)
        return np.asarray(t, dtype=np.float32)

    def linear_f32(self, base: str) -> np.ndarray:
        """Weight of linear ``base`` as float32: stored as such, or dequantised from its W4 pair
        (the converter also quantises the router gate; the reference loader dequantises it,
        src/model_glm52.cpp:169-193)."""
        if self.has(base + ".weight"):
            return self.float_tensor(base + ".weight")
        from .quant import dequantize_w4_np
        q, s = self._w4(base)
        return dequantize_w4_np(np.asarray(q), np.asarray(s, np.float32), self.group_of(base))

    # ---- the MLP half of a layer -------------------------------------------------------
    def _w4(self, base: str):
        """(qweight uint8 [out, in/2], scales float32 [out, in/group]) of linear ``base``."""
        if not self.has(base + ".qweight"):
            raise KeyError(f"{base}: no .qweight/.scales pair (not a W4 checkpoint, or the converter "
                           "left this linear unquantised because its input dim is not group-aligned)")
        return self.tensor(base + ".qweight"), self.tensor(base + ".scales")

    def group_of(self, base: str) -> int:
        q, s = self._w4(base)
        return int(q.shape[1] * 2 // s.shape[1])

    def is_moe_layer(self, i: int) -> bool:
        return i >= int(self.config.get("first_k_dense_replace", 0))

    def load_moe_layer(self, i: int) -> dict:
        """Layer dict (numpy) in the shape glmserve_b200.synth / ops.MoELayer use."""
        c = self.config
        p = f"model.layers.{i}.mlp."
        E = int(c["n_routed_experts"])
        first = self._first(p + "experts.0.gate_proj")
        group = self.group_of(first)
        gate = [self._w4(p + f"experts.{e}.gate_proj") for e in range(E)]
        up = [self._w4(p + f"experts.{e}.up_proj") for e in range(E)]
        down = [self._w4(p + f"experts.{e}.down_proj") for e in range(E)]
        I, hb = gate[0][0].shape
        router = p + ("gate" if self.has(p + "gate.weight") or self.has(p + "gate.qweight") else "router")
        L = dict(H=hb * 2, E=E, topk=int(c["num_experts_per_tok"]), I=int(I), Is=0, group=group,
                 norm_topk=bool(c.get("norm_topk_prob", True)),
                 routed_scale=float(c.get("routed_scaling_factor", 1.0)),
                 router_w=self.linear_f32(router), e_bias=None,
                 gate_q=np.stack([q for q, _ in gate]), gate_sc=np.stack([s for _, s in gate]),
                 up_q=np.stack([q for q, _ in up]), up_sc=np.stack([s for _, s in up]),
                 down_q=np.stack([q for q, _ in down]), down_sc=np.stack([s for _, s in down]))
        for bn in (p + "gate.e_score_correction_bias", p + "e_score_correction_bias"):
            if self.has(bn):
                L["e_bias"] = self.float_tensor(bn)
                break
        for sh in (p + "shared_experts.", p + "shared_expert."):
            if self.has(sh + "gate_proj.qweight"):
                (L["sg_q"], L["sg_sc"]), (L["su_q"], L["su_sc"]), (L["sd_q"], L["sd_sc"]) = (
                    self._w4(sh + "gate_proj"), self._w4(sh + "up_proj"), self._w4(sh + "down_proj"))
                L["Is"] = int(L["sg_q"].shape[0])
                break
        return L

    def _first(self, base: str) -> str:
        self._w4(base)
        return base

    def load_dense_mlp(self, i: int):
        """(gate_q, gate_sc, up_q, up_sc, down_q, down_sc) of a dense layer (``ops.DenseMLP``)."""
        p = f"model.layers.{i}.mlp."
        return (*self._w4(p + "gate_proj"), *self._w4(p + "up_proj"), *self._w4(p + "down_proj"))


def scales_fp16_report(L: dict) -> dict:
    """The kernels keep scales in fp16 (the converter writes fp32): the largest relative change
    that rounding makes, per tensor.  0 means the checkpoint's scales are fp16-representable."""
    rep = {}
    for k, v in L.items():
        if k.endswith("_sc") and v is not None:
            s = np.asarray(v, np.float32)
            r = s.astype(np.float16).astype(np.float32)
            rep[k] = float(np.max(np.abs(r - s) / np.maximum(np.abs(s), 1e-30)))
    return rep


def prepack_layer_np(L: dict) -> dict:
    """Tile streams of a layer dict (numpy twin of gsb_prepack_*; group 128 shapes only)."""
    from .quant import prepack_np
    out = {}
    if L["group"] != 128 or L["H"] % 512 or L["I"] % 512:
        return out
    f16 = lambda a: np.asarray(a, np.float32).astype(np.float16)
    out["gate_up_packed"] = prepack_np(L["gate_q"], f16(L["gate_sc"]), L["up_q"], f16(L["up_sc"]))
    out["down_packed"] = prepack_np(L["down_q"], f16(L["down_sc"]))
    if L.get("sg_q") is not None and L["Is"] % 512 == 0:
        out["shared_gate_up_packed"] = prepack_np(L["sg_q"][None], f16(L["sg_sc"])[None], L["su_q"][None],
                                                  f16(L["su_sc"])[None])
        out["shared_down_packed"] = prepack_np(L["sd_q"][None], f16(L["sd_sc"])[None])
    return out


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="gather (and prepack) one layer's MLP from a W4 checkpoint")
    ap.add_argument("model_dir")
    ap.add_argument("--layer", type=int, required=True)
    ap.add_argument("--out", required=True, help=".npz to write")
    a = ap.parse_args(argv)
    ck = Checkpoint(a.model_dir)
    if ck.is_moe_layer(a.layer):
        L = ck.load_moe_layer(a.layer)
        arrays = {k: v for k, v in L.items() if isinstance(v, np.ndarray)}
        arrays.update(prepack_layer_np(L))
        meta = {k: v for k, v in L.items() if not isinstance(v, np.ndarray) and v is not None}
        print("moe layer", a.layer, meta, "scale fp16 rounding", scales_fp16_report(L))
    else:
        names = ("gate_q", "gate_sc", "up_q", "up_sc", "down_q", "down_sc")
        arrays = dict(zip(names, ck.load_dense_mlp(a.layer)))
        meta = {"dense": True}
        print("dense layer", a.layer)
    np.savez(a.out, meta=json.dumps(meta), **arrays)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
