"""Writes the fixtures under tests/golden/ from the reference checkout.

Run in a container that has the reference mounted:

    python tests/golden/make_golden.py /root/reference

reference_decode.json: the reference's own known-answer file for its decode
seam (triton/examples/reference/reference_decode.json, produced by its DXIR
interpreter over maestro/.../ReferenceDecodeGraph.kt): five decode steps with
their logits.  It is re-serialised unchanged (inputs and outputs only) so the
tests can run where the reference is not mounted.
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


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
