"""Writes the fixtures under tests/golden/ from the reference checkout.

Run in a container that has the reference mounted:

    python tests/golden/make_golden.py <path of the reference checkout>

reference_decode.json: the reference's own known-answer file for its decode
seam (triton/examples/reference/reference_decode.json, produced by its DXIR
interpreter over maestro/.../ReferenceDecodeGraph.kt): five decode steps with
their logits.  It is re-serialised unchanged (inputs and outputs only) so the
tests can run where the reference is not mounted.

tiny_granite.npz / tiny_granite.json: the reference's tiny Granite checkpoint
(ir/src/jvmTest/resources/io/tlaloc/ir/inference/tiny_granite/: a 3-layer Llama-style decoder with the four
Granite scalars), its tensors as f32 arrays, with the two known answers the reference holds for it: every logit
at every position of two prompts from transformers' own GraniteForCausalLM (granite_modeling_logits.json, the
oracle of HfGraniteParityTest.theReferenceIsTransformersGraniteCode) and the greedy continuations with their
smallest top-1 margins (tiny_granite/greedy.json).  They pin the RMSNorm, RoPE, SwiGLU, grouped-query attention
and layer structure of the CPU oracle's decode step, which reference_decode.json does not exercise.
"""
import json
import os
import sys


def main(ref_root: str) -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(ref_root, "triton/examples/reference/reference_decode.json")) as f:
        src = json.load(f)
    out = {
        "origin": "triton/examples/reference/reference_decode.json (" + src.get("source", "") + ")",
        "model": {"vocab": 11, "d_model": 8, "num_heads": 4, "num_kv_heads": 2, "head_dim": 2, "num_blocks": 6,
                  "block_size": 2, "lcg": "s = s*1664525 + 1013904223 mod 2^32; w = f32((s>>>8)/2^24) - 0.5f",
                  "seeds": {"embed": 1, "q": 2, "k": 3, "v": 4, "head": 5}},
        "steps": src["steps"],
    }
    with open(os.path.join(here, "reference_decode.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote reference_decode.json with", len(out["steps"]), "steps")
    granite(ref_root, here)


def granite(ref_root: str, here: str) -> None:
    import numpy as np
    from safetensors import safe_open

    res = os.path.join(ref_root, "ir/src/jvmTest/resources/io/tlaloc/ir/inference")
    with safe_open(os.path.join(res, "tiny_granite/model.safetensors"), "np") as f:
        tensors = {k: f.get_tensor(k).astype(np.float32) for k in f.keys()}
    np.savez_compressed(os.path.join(here, "tiny_granite.npz"), **tensors)
    with open(os.path.join(res, "tiny_granite/config.json")) as f:
        config = json.load(f)
    with open(os.path.join(res, "tiny_granite/greedy.json")) as f:
        greedy = json.load(f)
    with open(os.path.join(res, "granite_modeling_logits.json")) as f:
        logits = json.load(f)
    out = {"origin": "ir/src/jvmTest/resources/io/tlaloc/ir/inference/{tiny_granite/*, granite_modeling_logits.json}",
           "config": config, "greedy": greedy, "modeling_logits": logits}
    with open(os.path.join(here, "tiny_granite.json"), "w") as f:
        json.dump(out, f)
    print("wrote tiny_granite.npz with", len(tensors), "tensors and tiny_granite.json")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
