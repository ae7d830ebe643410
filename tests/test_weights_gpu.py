"""An exported artifact's staged weight files on the device: a decoder loaded from `tlaloc-serving.json` + raw files
computes what the same weights loaded from memory compute, and the negative control of the reference's serving checks
(triton/int8_wrong_axis.py, triton/verify.sh:686-738): the same model with its int8 codes quantized along the WRONG
axis must fail parity against the oracle's step on the right weights (needs a B200)."""
import numpy as np
import pytest
import torch

import oracle
from tlaloc_b200 import weights as W

pytestmark = pytest.mark.gpu


def run_steps(dec, sharding, tables, ids, steps, B, bs):
    outs = []
    for step in range(steps):
        pos = np.full(B, step, np.int32)
        dec.set_inputs(ids[step], pos, tables, pos + 1, sharding.slot_mapping(tables, pos, bs))
        dec.step()
        outs.append(dec.logits.cpu().numpy().copy())
    return outs


def test_decoder_from_staged_files_and_the_wrong_axis_control(tmp_path):
    from tlaloc_b200 import decoder as D
    from tlaloc_b200 import sharding

    shape = oracle.DecoderShape(num_layers=2, d_model=256, num_heads=4, num_kv_heads=2, head_dim=64, ffn=688, vocab=1024,
                                kv_dtype="bf16", head_quant=True)
    ow = oracle.make_weights(shape, seed=5)
    w = W.DecoderWeights(embed=ow.embed, layers=ow.layers, final_norm=ow.final_norm, head=ow.head)
    model = {"vocabSize": 1024, "hiddenSize": 256, "numHeads": 4, "numKvHeads": 2, "headDim": 64, "blockSize": 16,
             "dtype": "bf16", "kvDtype": "bf16"}
    W.write_staged(str(tmp_path), w, model)
    staged = W.StagedWeights(str(tmp_path))
    assert staged.verify() == []
    cfg = D.DecoderConfig(**D.TINY, kv_dtype=torch.bfloat16, head_quant=True, max_positions=64)
    B, bs, M, steps = 4, 16, 3, 6
    rng = np.random.default_rng(0)
    tables = (1 + rng.permutation(B * M)).reshape(B, M).astype(np.int32)
    ids = [rng.integers(0, 1024, size=B).astype(np.int32) for _ in range(steps)]

    def decoder(weights):
        dec = D.Decoder(cfg, B, 1 + B * M, M)
        dec.load_host_weights(weights)
        return dec

    from_memory = run_steps(decoder(w), sharding, tables, ids, steps, B, bs)
    from_files = run_steps(decoder(staged.decoder_weights()), sharding, tables, ids, steps, B, bs)
    for a, b in zip(from_memory, from_files):
        assert np.array_equal(a, b)
    # the oracle's step on the right weights
    kp = [np.zeros((1 + B * M, bs, 2, 64), np.float32) for _ in range(2)]
    vp = [np.zeros_like(a) for a in kp]
    want = []
    for step in range(steps):
        pos = np.full(B, step, np.int32)
        want.append(oracle.decode_step(shape, ow, kp, vp, ids[step], pos, tables, pos + 1, sharding.slot_mapping(tables, pos, bs)))
    tol = lambda x: 2e-3 + 1e-2 * np.abs(x).max(axis=1, keepdims=True)
    assert all(np.all(np.abs(g - x) <= tol(x)) for g, x in zip(from_files, want))
    # the negative control: every projection quantized again per INPUT channel, scales left per output channel
    bad = staged.decoder_weights()
    for lw in bad.layers:
        for k in W.PROJECTIONS:
            codes, scales = lw[k]
            weight = codes.astype(np.float32) * scales[None, :]
            s_in = np.abs(weight).max(axis=1) / 127.0
            s_in[s_in == 0] = 1.0
            lw[k] = (np.clip(np.rint(weight / s_in[:, None]), -127, 127).astype(np.int8), scales)
    wrong = run_steps(decoder(bad), sharding, tables, ids, steps, B, bs)
    worst = max(float((np.abs(g - x) / tol(x)).max()) for g, x in zip(wrong, want))
    assert worst > 5.0, f"wrong-axis weights stayed within {worst:.1f}x of the tolerance: the parity check cannot see them"
