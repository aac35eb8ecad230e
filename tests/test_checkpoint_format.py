"""On-disk W4 checkpoint format (the reference converter's output,
tools/convert_hf_to_glmserve.py:216-251 and :323-380) through glmserve_b200.checkpoint.
The fixture under tests/golden/tiny_w4_ckpt was written by the reference's own tools
(tests/golden/make_w4_checkpoint_fixture.py); expected.npz holds GLM52Model::moe_mlp's output."""
import os

import numpy as np
import pytest

import oracle
from glmserve_b200.checkpoint import (Checkpoint, SafetensorsFile, prepack_layer_np, scales_fp16_report,
                                      write_safetensors, main as checkpoint_main)
from glmserve_b200.quant import dequantize_w4_np, prepack_np, quantize_w4_np
from glmserve_b200.synth import make_layer_np

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_w4_ckpt")


@pytest.fixture(scope="module")
def ck():
    return Checkpoint(FIX)


def test_moe_layer_is_gathered_from_per_expert_tensors(ck):
    L = ck.load_moe_layer(2)
    c = ck.config
    assert (L["H"], L["E"], L["topk"], L["I"], L["Is"], L["group"]) == (
        c["hidden_size"], c["n_routed_experts"], c["num_experts_per_tok"], c["moe_intermediate_size"],
        c["moe_intermediate_size"] * c["n_shared_experts"], 16)
    assert L["norm_topk"] is True and L["routed_scale"] == 2.5
    assert L["gate_q"].shape == (8, 48, 32) and L["gate_q"].dtype == np.uint8
    assert L["down_q"].shape == (8, 64, 24) and L["down_sc"].shape == (8, 64, 3)
    assert L["router_w"].shape == (8, 64) and L["e_bias"].shape == (8,)
    # expert 5 of the gathered array is the file's tensor of that name
    q = SafetensorsFile(os.path.join(FIX, "model.safetensors")).tensor("model.layers.2.mlp.experts.5.up_proj.qweight")
    assert np.array_equal(L["up_q"][5], q)
    assert ck.is_moe_layer(2) and not ck.is_moe_layer(0)


def test_quantiser_twin_reproduces_the_converter(ck):
    """quantize_w4_np on the fp32 originals gives the converter's nibbles exactly, and its scales
    are the converter's rounded to fp16."""
    fp = SafetensorsFile(os.path.join(FIX, "fp", "fp_subset.safetensors"))
    checked = 0
    for name in fp.names():
        if not name.endswith("_proj.weight") and not name.endswith("mlp.gate.weight"):
            continue
        base = name[:-len(".weight")]
        q_file, s_file = ck.tensor(base + ".qweight"), ck.tensor(base + ".scales")
        q, s16 = quantize_w4_np(np.asarray(fp.tensor(name), np.float32), 16)
        assert np.array_equal(q, q_file), name
        assert np.array_equal(s16, np.asarray(s_file).astype(np.float16).astype(np.float32)), name
        checked += 1
    assert checked >= 8


def test_loaded_layer_through_the_oracle_equals_the_reference_output(ck):
    L = ck.load_moe_layer(2)
    e = np.load(os.path.join(FIX, "expected.npz"))
    r = oracle.moe_layer_w4(e["x"], L)
    assert r["ties"] == 0
    assert np.array_equal(r["out"], e["out_ref"])


def test_router_gate_quantised_by_the_converter_is_dequantised(ck):
    q, s = ck.tensor("model.layers.2.mlp.gate.qweight"), ck.tensor("model.layers.2.mlp.gate.scales")
    assert np.array_equal(ck.linear_f32("model.layers.2.mlp.gate"), dequantize_w4_np(np.asarray(q), np.asarray(s), 16))


def test_dense_layer_tensors(ck):
    gq, gs, uq, us, dq, ds = ck.load_dense_mlp(0)
    assert gq.shape == (128, 32) and gs.shape == (128, 4) and dq.shape == (64, 64) and ds.shape == (64, 8)
    with pytest.raises(KeyError):
        ck.load_dense_mlp(2)


def test_scales_fp16_report_and_missing_pairs(ck):
    rep = scales_fp16_report(ck.load_moe_layer(2))
    assert set(rep) == {"gate_sc", "up_sc", "down_sc", "sg_sc", "su_sc", "sd_sc"}
    assert all(0 < v < 2 ** -10 for v in rep.values())       # fp32 scales: rounding is visible but < 1 ulp of fp16
    with pytest.raises(KeyError):
        ck._w4("model.layers.2.mlp.experts.99.gate_proj")


def test_safetensors_round_trip_with_bf16_and_sharded_index(tmp_path):
    rng = np.random.default_rng(0)
    a = rng.integers(0, 256, (3, 10), dtype=np.uint8)
    b = rng.standard_normal((4, 6)).astype(np.float32)
    bits = (b.view(np.uint32) >> 16).astype(np.uint16)
    write_safetensors(str(tmp_path / "s0.safetensors"), {"a.qweight": a, "h": b.astype(np.float16)})
    write_safetensors(str(tmp_path / "s1.safetensors"), {"w": ("BF16", bits), "i": np.arange(5, dtype=np.int64)})
    (tmp_path / "config.json").write_text("{}")
    c = Checkpoint(str(tmp_path))                     # no index file: shards are scanned
    assert np.array_equal(c.tensor("a.qweight"), a) and c.dtype("w") == "BF16"
    assert np.array_equal(c.float_tensor("w"), (bits.astype(np.uint32) << 16).view(np.float32))
    assert np.array_equal(c.float_tensor("h"), b.astype(np.float16).astype(np.float32))
    (tmp_path / "model.safetensors.index.json").write_text(
        '{"weight_map": {"a.qweight": "s0.safetensors", "w": "s1.safetensors"}}')
    c2 = Checkpoint(str(tmp_path))
    assert c2.has("w") and not c2.has("i") and np.array_equal(c2.tensor("a.qweight"), a)


def test_prepack_tool_writes_tile_streams_for_group_128_layers(tmp_path):
    """A GLM-shaped (small) layer written in the converter's naming, read back and prepacked:
    the streams equal prepack_np on the original arrays."""
    cfg = dict(H=512, E=2, topk=1, I=512, Is=512, group=128)
    L = make_layer_np(cfg, seed=3)
    t = {}
    p = "model.layers.3.mlp."
    for e in range(2):
        for nm in ("gate", "up", "down"):
            t[p + f"experts.{e}.{nm}_proj.qweight"] = L[nm + "_q"][e]
            t[p + f"experts.{e}.{nm}_proj.scales"] = L[nm + "_sc"][e].astype(np.float32)
    for nm, key in (("gate", "sg"), ("up", "su"), ("down", "sd")):
        t[p + f"shared_experts.{nm}_proj.qweight"] = L[key + "_q"]
        t[p + f"shared_experts.{nm}_proj.scales"] = L[key + "_sc"].astype(np.float32)
    t[p + "gate.weight"] = L["router_w"].astype(np.float32)
    t[p + "gate.e_score_correction_bias"] = L["e_bias"].astype(np.float32)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    (tmp_path / "config.json").write_text(
        '{"n_routed_experts": 2, "num_experts_per_tok": 1, "first_k_dense_replace": 3, '
        '"norm_topk_prob": true, "routed_scaling_factor": 2.5}')
    out = str(tmp_path / "layer3.npz")
    assert checkpoint_main([str(tmp_path), "--layer", "3", "--out", out]) == 0
    z = np.load(out)
    f16 = lambda a: a.astype(np.float16)
    assert np.array_equal(z["gate_up_packed"], prepack_np(L["gate_q"], f16(L["gate_sc"]), L["up_q"], f16(L["up_sc"])))
    assert np.array_equal(z["down_packed"], prepack_np(L["down_q"], f16(L["down_sc"])))
    assert np.array_equal(z["shared_down_packed"], prepack_np(L["sd_q"][None], f16(L["sd_sc"])[None]))
    assert prepack_layer_np(Checkpoint(FIX).load_moe_layer(2)) == {}   # group 16: direct-layout kernels only
