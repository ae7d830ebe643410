"""The CPU oracle's decode step pinned on the reference's tiny Granite checkpoint (tests/golden/tiny_granite.*, copied
from ir/src/jvmTest/resources/io/tlaloc/ir/inference/ by tests/golden/make_golden.py): a 3-layer Llama-style decoder
(hidden 32, 4 query / 2 KV heads, FFN 48, vocab 64) with Granite's four scalars.  Two known answers of the reference:
  - every logit at every position of two prompts, computed by transformers' own GraniteForCausalLM
    (granite_modeling_logits.json; the reference holds its own dense forward pass to it at 2e-4,
    HfGraniteParityTest.kt:160-178, and its decode graph to that at the same bar, :186-230);
  - the greedy continuations of five prompts with their smallest top-1 margins (tiny_granite/greedy.json, :74-99).
These reach what reference_decode.json does not: RMSNorm, RoPE (rotate_half, duplicated tables), SwiGLU, grouped-query
attention over several pages, residual adds, the final norm."""
import json
import os

import numpy as np

import oracle

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 2e-4  # HfGraniteParityTest.kt:341


def load():
    fx = json.load(open(os.path.join(HERE, "tiny_granite.json")))
    t = dict(np.load(os.path.join(HERE, "tiny_granite.npz")))
    c = fx["config"]
    hd = c["hidden_size"] // c["num_attention_heads"]
    shape = oracle.DecoderShape(
        num_layers=c["num_hidden_layers"], d_model=c["hidden_size"], num_heads=c["num_attention_heads"],
        num_kv_heads=c["num_key_value_heads"], head_dim=hd, ffn=c["intermediate_size"], vocab=c["vocab_size"],
        rms_eps=c["rms_norm_eps"], rope_theta=c["rope_parameters"]["rope_theta"], block_size=4, weight_dtype="f32",
        kv_dtype="f32", head_quant=False, embed_scale=c["embedding_multiplier"], attention_scale=c["attention_multiplier"],
        residual_multiplier=c["residual_multiplier"], logit_multiplier=1.0 / c["logits_scaling"])
    w = oracle.DecoderWeights(embed=t["model.embed_tokens.weight"])
    for l in range(shape.num_layers):
        p = f"model.layers.{l}."
        io = lambda name: np.ascontiguousarray(t[p + name + ".weight"].T)  # checkpoint [out, in] -> staged [in, out]
        w.layers.append({"q": io("self_attn.q_proj"), "k": io("self_attn.k_proj"), "v": io("self_attn.v_proj"),
                         "o": io("self_attn.o_proj"), "gate": io("mlp.gate_proj"), "up": io("mlp.up_proj"),
                         "down": io("mlp.down_proj"), "ln1": t[p + "input_layernorm.weight"],
                         "ln2": t[p + "post_attention_layernorm.weight"]})
    w.final_norm = t["model.norm.weight"]
    w.head = np.ascontiguousarray(t["lm_head.weight"].T)
    return fx, shape, w


class Session:
    """One sequence decoded token by token through the paged step (pages of 4, permuted)."""

    def __init__(self, shape, w, max_len=48):
        self.shape, self.w, bs = shape, w, shape.block_size
        self.M = max_len // bs
        nb = 1 + self.M
        self.table = (1 + np.random.default_rng(1).permutation(self.M)).astype(np.int32)[None, :]
        self.kp = [np.zeros((nb, bs, shape.num_kv_heads, shape.head_dim), np.float32) for _ in range(shape.num_layers)]
        self.vp = [np.zeros_like(a) for a in self.kp]
        self.pos = 0

    def feed(self, token):
        bs = self.shape.block_size
        slot = np.array([self.table[0, self.pos // bs] * bs + self.pos % bs], np.int32)
        logits = oracle.decode_step(self.shape, self.w, self.kp, self.vp, np.array([token], np.int32),
                                    np.array([self.pos], np.int32), self.table, np.array([self.pos + 1], np.int32), slot)
        self.pos += 1
        return logits[0]


def test_every_logit_of_transformers_granite_code():
    fx, shape, w = load()
    worst = 0.0
    for p in fx["modeling_logits"]["prompts"]:
        s = Session(shape, w)
        for t, tok in enumerate(p["ids"]):
            got = s.feed(tok)
            err = np.abs(got.astype(np.float64) - np.asarray(p["logits"][t]))
            worst = max(worst, float(err.max()))
            assert err.max() <= TOL, (p["ids"], t, float(err.max()))
    print(f"oracle against modeling_granite.py: worst |logit difference| {worst:.2e}")


def test_greedy_continuations_and_their_margins():
    fx, shape, w = load()
    for name, (prompt, want_ids, want_margin) in fx["greedy"].items():
        s = Session(shape, w)
        for tok in prompt[:-1]:
            s.feed(tok)
        tok, got_ids, margin = prompt[-1], [], np.inf
        for _ in want_ids:
            l = s.feed(tok)
            order = np.argsort(-l, kind="stable")
            margin = min(margin, float(l[order[0]] - l[order[1]]))
            tok = int(oracle.argmax(l[None, :])[0])
            got_ids.append(tok)
        assert got_ids == want_ids, name
        assert abs(margin - want_margin) <= 2 * TOL, (name, margin, want_margin)


def test_each_scalar_matters():
    """HfGraniteParityTest.eachMultiplierMovesTheLogits: dropping any one of the four moves the logits far past TOL."""
    fx, shape, w = load()
    ids = fx["modeling_logits"]["prompts"][1]["ids"]

    def last(sh):
        s = Session(sh, w)
        for tok in ids:
            out = s.feed(tok)
        return out

    base = last(shape)
    import dataclasses
    for field, off in [("embed_scale", None), ("attention_scale", None), ("residual_multiplier", 1.0), ("logit_multiplier", 1.0)]:
        moved = np.abs(last(dataclasses.replace(shape, **{field: off})) - base).max()
        assert moved > 100 * TOL, (field, float(moved))
