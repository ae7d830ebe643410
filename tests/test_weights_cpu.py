"""Host-side weights: the product's int8 quantizer against the oracle's restatement of HfStagedWeights.quantize
(bit for bit), the staged weight files + manifest round trip, the wrong-axis negative control
(triton/int8_wrong_axis.py, triton/verify.sh:686-738: a model quantized along the input axis must FAIL a quality
check), and the safetensors reader."""
import json
import os
import struct

import numpy as np
import pytest

import oracle
from tlaloc_b200 import weights as W


def test_quantizer_is_bit_equal_to_the_oracles():
    rng = np.random.default_rng(0)
    for shape in [(1, 1), (7, 5), (64, 256), (688, 256), (1024, 4096)]:
        w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
        w[0, :] = 0.0  # a row of zeros: scale 1, codes 0
        if shape[1] >= 4:
            w[-1, :4] = [0.5, 1.5, 2.5, -2.5]  # with max 127 these would be exact halves
            w[-1, -1] = 127.0
        codes, scales = W.quantize_int8(w)
        ocodes, oscales = oracle.quantize_int8(w)
        assert codes.dtype == np.int8 and codes.shape == (shape[1], shape[0]) and scales.shape == (shape[0],)
        assert np.array_equal(codes, ocodes) and np.array_equal(scales.view(np.uint32), oscales.view(np.uint32))
        assert scales[0] == 1.0 and not codes[:, 0].any()
    w = np.array([[0.5, 1.5, 2.5, -2.5, 3.5, 127.0]], np.float32)
    codes, scales = W.quantize_int8(w)
    assert scales[0] == 1.0 and codes[:, 0].tolist() == [0, 2, 2, -2, 4, 127]  # halves go to even, not away from zero
    assert np.abs(W.dequantize_int8(codes, scales) - w).max() <= 0.5
    assert np.array_equal(W.snap_bf16(np.array([1.00390625, 1.01171875, np.inf], np.float32)),
                          oracle.snap_bf16(np.array([1.00390625, 1.01171875, np.inf], np.float32)))
    x = rng.standard_normal(4096).astype(np.float32)
    assert np.array_equal(W.f32_to_bf16_bits(x), oracle.bf16_bits(x))


def _tiny(seed=0, head_quant=True):
    shape = oracle.DecoderShape(num_layers=2, d_model=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn=96, vocab=128,
                                kv_dtype="bf16", head_quant=head_quant)
    ow = oracle.make_weights(shape, seed=seed)
    return shape, W.DecoderWeights(embed=ow.embed, layers=ow.layers, final_norm=ow.final_norm, head=ow.head)


@pytest.mark.parametrize("head_quant", [True, False])
def test_staged_files_round_trip_and_are_checked(tmp_path, head_quant):
    shape, w = _tiny(head_quant=head_quant)
    model = {"vocabSize": 128, "hiddenSize": 64, "numHeads": 4, "numKvHeads": 2, "headDim": 16, "blockSize": 16,
             "dtype": "bf16", "kvDtype": "bf16"}
    W.write_staged(str(tmp_path), w, model)
    st = W.StagedWeights(str(tmp_path))
    assert st.model["numLayers"] == 2 and st.verify() == []
    names = list(st.files)
    assert names[:3] == ["embedTokens", "inputNorm0", "qProj0"] and "qProj0Scale" in names and names[-1] in ("lmHead", "lmHeadScale")
    assert st.files["qProj1"].dtype == "i8" and st.files["qProj1"].dims == [64, 64]
    back = st.decoder_weights()
    assert np.array_equal(back.embed, w.embed) and np.array_equal(back.final_norm, w.final_norm)
    for a, b in zip(back.layers, w.layers):
        for k in W.PROJECTIONS:
            assert np.array_equal(a[k][0], b[k][0]) and np.array_equal(a[k][1], b[k][1])
        assert np.array_equal(a["ln1"], b["ln1"]) and np.array_equal(a["ln2"], b["ln2"])
    if head_quant:
        assert np.array_equal(back.head[0], w.head[0]) and np.array_equal(back.head[1], w.head[1])
    else:
        assert np.array_equal(back.head, w.head)
    # a changed byte shows in verify(); a truncated file and a lying manifest are refused on read
    path = os.path.join(str(tmp_path), st.files["kProj0"].path)
    raw = bytearray(open(path, "rb").read())
    raw[3] ^= 1
    open(path, "wb").write(raw)
    assert W.StagedWeights(str(tmp_path)).verify() == ["kProj0"]
    open(path, "wb").write(raw[:-1])
    with pytest.raises(ValueError, match="bytes on disk"):
        W.StagedWeights(str(tmp_path)).read("kProj0")
    man = json.load(open(os.path.join(str(tmp_path), W.MANIFEST)))
    man["weights"]["table"][2]["dims"] = [64, 63]
    json.dump(man, open(os.path.join(str(tmp_path), W.MANIFEST), "w"))
    with pytest.raises(ValueError, match="states"):
        W.StagedWeights(str(tmp_path))
    man["weights"] = {"format": "embedded", "path": None, "embedded": True, "table": []}
    json.dump(man, open(os.path.join(str(tmp_path), W.MANIFEST), "w"))
    with pytest.raises(ValueError, match="staged"):
        W.StagedWeights(str(tmp_path))


def wrong_axis(codes, scales):
    """What triton/int8_wrong_axis.py does to one projection: quantize again with one scale per INPUT channel while
    the scale slot keeps its per-output values."""
    weight = codes.astype(np.float32) * scales[None, :]
    s_in = np.abs(weight).max(axis=1) / 127.0
    s_in[s_in == 0] = 1.0
    return np.clip(np.rint(weight / s_in[:, None]), -127, 127).astype(np.int8)


def test_wrong_axis_quantization_fails_parity_and_the_right_axis_passes():
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((256, 512)) * 0.02 * rng.uniform(0.2, 5.0, size=(256, 1))).astype(np.float32)  # rows of unequal size
    x = oracle.snap_bf16(rng.standard_normal((8, 512)).astype(np.float32))
    want = x.astype(np.float64) @ w.astype(np.float64).T
    codes, scales = W.quantize_int8(w)
    good = oracle.proj_int8(x, codes, scales)
    bad = oracle.proj_int8(x, wrong_axis(codes, scales), scales)
    mag = np.abs(want).max()
    assert np.abs(good - want).max() <= 1e-2 * mag
    assert np.abs(bad - want).max() >= 0.2 * mag  # nowhere near: the quality check must fail on it


def test_safetensors_reader_and_checkpoint_quantization(tmp_path):
    rng = np.random.default_rng(4)
    tensors = {"model.embed_tokens.weight": rng.standard_normal((32, 16)).astype(np.float32),
               "model.norm.weight": rng.standard_normal(16).astype(np.float32),
               "lm_head.weight": rng.standard_normal((32, 16)).astype(np.float32)}
    for l in range(2):
        p = f"model.layers.{l}."
        for hf, shp in [("self_attn.q_proj", (16, 16)), ("self_attn.k_proj", (8, 16)), ("self_attn.v_proj", (8, 16)),
                        ("self_attn.o_proj", (16, 16)), ("mlp.gate_proj", (24, 16)), ("mlp.up_proj", (24, 16)), ("mlp.down_proj", (16, 24))]:
            tensors[p + hf + ".weight"] = rng.standard_normal(shp).astype(np.float32)
        tensors[p + "input_layernorm.weight"] = rng.standard_normal(16).astype(np.float32)
        tensors[p + "post_attention_layernorm.weight"] = rng.standard_normal(16).astype(np.float32)
    # a file by hand: two tensors stored as bf16 and f16, the rest f32
    header, blobs, off = {}, [], 0
    for i, (name, a) in enumerate(tensors.items()):
        if i == 0:
            raw, dt = W.f32_to_bf16_bits(a).astype("<u2").tobytes(), "BF16"
        elif i == 1:
            raw, dt = a.astype("<f2").tobytes(), "F16"
        else:
            raw, dt = a.astype("<f4").tobytes(), "F32"
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    path = os.path.join(str(tmp_path), "model.safetensors")
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    got = W.read_safetensors(path)
    for i, (name, a) in enumerate(tensors.items()):
        want = W.snap_bf16(a) if i == 0 else a.astype(np.float16).astype(np.float32) if i == 1 else a
        assert np.array_equal(got[name], want), name
    try:  # the safetensors package, where installed, agrees on an f32 tensor (its NumPy reader has no bf16)
        from safetensors import safe_open
    except ImportError:
        safe_open = None
    if safe_open is not None:
        with safe_open(path, framework="np") as f:
            assert np.array_equal(f.get_tensor("lm_head.weight"), got["lm_head.weight"])
    w = W.quantize_checkpoint(got, 2, head_quant=False)
    assert w.layers[1]["down"][0].shape == (24, 16) and w.layers[1]["down"][0].dtype == np.int8
    assert np.array_equal(w.layers[0]["q"][0], oracle.quantize_int8(got["model.layers.0.self_attn.q_proj.weight"])[0])
    assert w.head.shape == (16, 32) and np.array_equal(w.head, oracle.snap_bf16(got["lm_head.weight"].T))
