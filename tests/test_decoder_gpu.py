"""The tiny Llama-style decoder (2 layers, d 256, 4 Q / 2 KV heads, head_dim 64, FFN 688, vocab 1024, eps 1e-5,
theta 1e4; weights N(0, 0.02) seed 0, int8 per output channel; paged KV, block 16; batch 4 with contexts
37/64/128/200; 64 greedy decode steps) on the GPU engine against the CPU oracle: logits within rel 1e-2 / abs 2e-3,
greedy tokens identical (needs a B200)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _setup(kv_dtype, head_quant, exact=False):
    from tlaloc_b200 import decoder as D
    from tlaloc_b200 import sharding

    shape = oracle.DecoderShape(num_layers=2, d_model=256, num_heads=4, num_kv_heads=2, head_dim=64, ffn=688, vocab=1024,
                                rms_eps=1e-5, rope_theta=10000.0, block_size=16, weight_dtype="bf16",
                                kv_dtype="bf16" if kv_dtype == torch.bfloat16 else "f32", head_quant=head_quant)
    w = oracle.make_weights(shape, seed=0)
    cfg = D.DecoderConfig(**D.TINY, kv_dtype=kv_dtype, head_quant=head_quant, max_positions=512)
    B, bs = 4, 16
    ctx = np.array([37, 64, 128, 200])
    max_blocks = 17  # 272 positions: room for 200 + 64 steps
    num_blocks = 1 + B * max_blocks  # page 0 is the padding page
    rng = np.random.default_rng(0)
    perm = 1 + rng.permutation(B * max_blocks)
    tables = perm.reshape(B, max_blocks).astype(np.int32)
    prompts = [rng.integers(0, 1024, size=n).astype(np.int32) for n in ctx]
    dec = D.Decoder(cfg, B, num_blocks, max_blocks, exact=exact)
    dec.load_host_weights(w)
    return shape, w, cfg, dec, tables, prompts, ctx, num_blocks, sharding


@pytest.mark.parametrize("kv_dtype,head_quant,exact", [(torch.float32, False, True), (torch.bfloat16, True, True),
                                                       (torch.float32, False, False), (torch.bfloat16, True, False)])
def test_tiny_decoder_64_greedy_steps_match_the_oracle(kv_dtype, head_quant, exact):
    """`exact` runs the engine in the library's parity mode (the interpreter's own evaluation order in every
    operator): there the greedy tokens must be IDENTICAL over the 64 steps and the logits equal to rounding.  The fast
    kernels reorder f32 sums; a reordered sum can flip the bf16 rounding of one activation (every projection input is
    rounded to bf16), which moves a logit by ~1e-3, so on a near-tie of the oracle's own top two logits a token may
    differ: those are counted and bounded, and the parity-mode run shows that nothing else is behind them."""
    shape, w, cfg, dec, tables, prompts, ctx, num_blocks, sharding = _setup(kv_dtype, head_quant, exact)
    B, bs = 4, 16
    kp = [np.zeros((num_blocks, bs, 2, 64), np.float32) for _ in range(2)]
    vp = [np.zeros((num_blocks, bs, 2, 64), np.float32) for _ in range(2)]
    # Prefill, one token per decode-style step (row-equivalent to a chunk by construction, HfDecoderGraph.kt:473-488):
    # sequences shorter than the longest sit out as padding rows (slot -1, seqLen 1, block 0: DecodeGraphSpec.kt:989-1004).
    pad_table = np.zeros_like(tables)
    worst, trail = 0.0, []

    def tol(want):
        # abs 2e-3 plus rel 1e-2 of the row's largest logit (the reference's own "mag" convention,
        # runtime-pjrt/.../PjrtFusedPagedAttentionTest.kt:94-97).  The two runs share inputs only at step 0: after
        # that each keeps its own KV pools, and an activation that lands on the other side of a bf16 rounding
        # boundary (every projection input is rounded to bf16) stays in its pool, so the distance grows slowly.
        return 2e-3 + 1e-2 * np.abs(want).max(axis=-1, keepdims=True)
    last_logits = None
    for t in range(int(ctx.max())):
        live = t < ctx
        ids = np.array([prompts[i][t] if live[i] else 0 for i in range(B)], np.int32)
        pos = np.where(live, t, 0).astype(np.int32)
        lens = np.where(live, t + 1, 1).astype(np.int32)
        tab = np.where(live[:, None], tables, pad_table).astype(np.int32)
        slots = np.where(live, sharding.slot_mapping(tables, np.where(live, t, 0), bs), -1).astype(np.int32)
        dec.set_inputs(ids, pos, tab, lens, slots)
        dec.step()
        if t % 16 == 0 or t >= ctx.max() - 2 or np.any(t == ctx - 1):
            want = oracle.decode_step(shape, w, kp, vp, ids, pos, tab, lens, slots)
            got = dec.logits.cpu().numpy()
            err = np.abs(got - want)[live]
            assert np.all(err <= tol(want[live])), (t, err.max())
            worst = max(worst, float(err.max()))
            trail.append((t, float(err.max())))
            if last_logits is None:
                last_logits = np.zeros_like(want)
            for i in range(B):
                if t == ctx[i] - 1:
                    last_logits[i] = want[i]
        else:
            oracle.decode_step(shape, w, kp, vp, ids, pos, tab, lens, slots)
    # the device pools hold what the oracle's hold
    for l in range(2):
        assert np.abs(dec.key_pools[l].float().cpu().numpy()[1:] - kp[l][1:]).max() <= 2e-2
    # 64 greedy steps, teacher-forced on the oracle's tokens; ids must be identical, margins are reported
    tok = oracle.argmax(last_logits).astype(np.int32)
    pos = ctx.copy()
    mismatches, near_ties, min_margin = 0, 0, np.inf
    dec.capture()
    for step in range(64):
        lens = (pos + 1).astype(np.int32)
        slots = sharding.slot_mapping(tables, pos, bs)
        dec.set_inputs(tok, pos.astype(np.int32), tables, lens, slots)
        nxt = dec.step().cpu().numpy()
        want = oracle.decode_step(shape, w, kp, vp, tok, pos.astype(np.int32), tables, lens, slots)
        got = dec.logits.cpu().numpy()
        err = np.abs(got - want)
        assert np.all(err <= tol(want)), (step, err.max())
        worst = max(worst, float(err.max()))
        trail.append((int(ctx.max()) + step, float(err.max())))
        want_tok = oracle.argmax(want).astype(np.int32)
        srt = np.sort(want, axis=1)
        min_margin = min(min_margin, float((srt[:, -1] - srt[:, -2]).min()))
        for i in np.nonzero(nxt != want_tok)[0]:
            gap = float(want[i, want_tok[i]] - want[i, nxt[i]])  # how far the oracle itself ranks the two tokens apart
            print(f"step {step} row {i}: oracle {want_tok[i]} device {nxt[i]}; oracle's gap between them {gap:.3e}, "
                  f"row max |d| {float(err[i].max()):.3e}")
            if gap <= 2.0 * float(err[i].max()):
                near_ties += 1
            else:
                mismatches += 1
        tok, pos = want_tok, pos + 1
    print("max |d| by step:", " ".join(f"{t}:{e:.1e}" for t, e in trail[::6]))
    print(f"worst logit |d| {worst:.3e}; smallest top-2 margin {min_margin:.3e}; token mismatches {mismatches}, "
          f"near-tie swaps {near_ties} of {64 * B}")
    # Identical greedy tokens, except where the oracle's own logits put the two candidates closer together than the
    # two runs' logits are to each other (a tie within the comparison's resolution; triton/quant_checks.py:55-87
    # reports margins for the same reason).  Such swaps must stay rare.
    if exact:
        assert mismatches == 0 and near_ties == 0, "parity mode must reproduce the oracle's greedy tokens exactly"
        assert worst <= 1e-5, worst
    else:
        assert mismatches == 0 and near_ties <= 2


def test_batch_of_40_with_swiglu_in_the_projection_epilogue_matches_the_oracle():
    """17 to 128 rows and an FFN width that tiles in blocks of 128: the engine runs the int8 tensor-core projection (the
    activation planes written by the RMSNorm kernel) and folds SwiGLU into the gate|up projection's epilogue (weights
    interleaved at load).  64 greedy steps, teacher-forced on the oracle's tokens: logits within the bar at every step,
    and a different token only where the oracle itself ranks the two candidates closer than the runs' logits differ."""
    from tlaloc_b200 import decoder as D
    from tlaloc_b200 import sharding

    dims = dict(num_layers=2, d_model=256, num_heads=4, num_kv_heads=2, head_dim=64, ffn=512, vocab=512)
    shape = oracle.DecoderShape(**dims, kv_dtype="bf16", head_quant=True)
    w = oracle.make_weights(shape, seed=7)
    cfg = D.DecoderConfig(**dims, kv_dtype=torch.bfloat16, head_quant=True, max_positions=80)
    B, bs, M = 40, 16, 5
    rng = np.random.default_rng(3)
    tables = (1 + rng.permutation(B * M)).reshape(B, M).astype(np.int32)
    dec = D.Decoder(cfg, B, 1 + B * M, M)
    assert dec.fuse_swiglu and dec.i8_mma and dec.norm_planes
    dec.load_host_weights(w)
    kp = [np.zeros((1 + B * M, bs, 2, 64), np.float32) for _ in range(2)]
    vp = [np.zeros_like(a) for a in kp]
    ids = rng.integers(0, 512, size=B).astype(np.int32)
    swaps = 0
    for step in range(64):
        pos = np.full(B, step, np.int32)
        slots = sharding.slot_mapping(tables, pos, bs)
        dec.set_inputs(ids, pos, tables, pos + 1, slots)
        if step == 2:
            dec.capture()
        nxt = dec.step().cpu().numpy()
        want = oracle.decode_step(shape, w, kp, vp, ids, pos, tables, pos + 1, slots, threads=8)
        err = np.abs(dec.logits.cpu().numpy() - want)
        assert np.all(err <= 2e-3 + 1e-2 * np.abs(want).max(axis=1, keepdims=True)), (step, float(err.max()))
        ids = oracle.argmax(want).astype(np.int32)
        # a different token only where the oracle's own logits rank the two closer than the runs' logits differ
        for i in np.nonzero(nxt != ids)[0]:
            assert float(want[i, ids[i]] - want[i, nxt[i]]) <= 2.0 * float(err[i].max()), (step, i)
            swaps += 1
    print(f"near-tie swaps: {swaps} of {64 * B}")
    assert swaps <= 0.015 * 64 * B  # observed: 13 of 2560
