"""Weights of the decode path on the host: the int8 per-output-channel quantizer, the staged weight files of an
exported serving artifact (`tlaloc-serving.json` + raw little-endian files), and Hugging Face safetensors.

What this follows in the reference:
  - quantizer: HfStagedWeights.quantize, ir/src/jvmMain/kotlin/io/tlaloc/ir/inference/HfStagedWeights.kt:396-461
    (INT8 arm :433-444): per output channel (a row of the checkpoint's [out, in]), scale = max|w| / 127 (1 for a row
    of zeros), code = clamp(rint(w / scale), -127, 127) with rint rounding halves to even, codes staged as [in, out];
  - staged files: one raw little-endian file per weight slot, listed in the manifest's `weights.table` with name,
    path, dtype tag, dims, byteLength and sha256 (maestro/.../serving/ServingManifest.kt:762-870; the int8 convention
    "codes i8 [in, out] followed by f32 scales [out] in the slot <name>Scale" as triton/int8_wrong_axis.py:42-50 reads it);
  - slot names: HfDecoderGraph.slotName, ir/.../inference/HfDecoderGraph.kt:285-380 (embedTokens, inputNorm<l>, qProj<l>,
    kProj<l>, vProj<l>, oProj<l>, postAttnNorm<l>, gateProj<l>, upProj<l>, downProj<l>, finalNorm, lmHead).

Everything here is host-side NumPy; the device never sees a float weight of a quantized projection.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from dataclasses import dataclass, field

import numpy as np

MANIFEST = "tlaloc-serving.json"
STAGED_FORMAT, STAGED_DIR = "staged", "weights"
_DTYPES = {"i8": np.int8, "f32": np.float32, "bf16": np.uint16, "i32": np.int32, "u8": np.uint8}
PROJECTIONS = ("q", "k", "v", "o", "gate", "up", "down")
_SLOT = {"q": "qProj", "k": "kProj", "v": "vProj", "o": "oProj", "gate": "gateProj", "up": "upProj", "down": "downProj"}
_HF = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
       "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}


# ---------------------------------------------------------------------------------------------- the quantizer

def quantize_int8(w_out_in) -> tuple[np.ndarray, np.ndarray]:
    """w [out, in] f32 -> (codes int8 [in, out], scales f32 [out]), exactly as the exporter quantizes a projection:
    every step in f32 except the rounding, which widens the f32 quotient to double and rounds halves to even."""
    w = np.ascontiguousarray(w_out_in, dtype=np.float32)
    if w.ndim != 2:
        raise ValueError(f"quantize_int8: a projection is [out, in], got shape {w.shape}")
    mx = np.abs(w).max(axis=1) if w.shape[1] else np.zeros(w.shape[0], np.float32)
    scales = np.where(mx == 0, np.float32(1), mx / np.float32(127)).astype(np.float32)
    q = (w / scales[:, None]).astype(np.float32)  # the f32 quotient
    codes = np.clip(np.rint(q.astype(np.float64)), -127.0, 127.0).astype(np.int8)
    return np.ascontiguousarray(codes.T), scales


def dequantize_int8(codes_in_out, scales) -> np.ndarray:
    """codes [in, out], scales [out] -> the f32 weight [out, in] the codes stand for."""
    return np.ascontiguousarray((codes_in_out.astype(np.float32) * np.asarray(scales, np.float32)[None, :]).T)


def snap_bf16(x) -> np.ndarray:
    """f32 values rounded to the nearest bf16 (ties to even), still as f32 (core/.../Bf16.kt:57-71)."""
    return bf16_to_f32(f32_to_bf16_bits(x))


def f32_to_bf16_bits(x) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((u >> 16) | 0x0040).astype(np.uint16), r)


def bf16_to_f32(bits) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------------------------------------- the decoder's weights

@dataclass
class DecoderWeights:
    """A Llama-style decoder in the staged layout: per projection int8 codes [in, out] + f32 scales [out]; the
    embedding table and (unless quantized) the head as f32 values; f32 norm gains."""

    embed: np.ndarray
    layers: list = field(default_factory=list)  # dicts: q, k, v, o, gate, up, down -> (codes, scales); ln1, ln2
    final_norm: np.ndarray | None = None
    head: tuple | np.ndarray | None = None  # (codes [d, vocab], scales [vocab]) or f32 [d, vocab]


def quantize_checkpoint(tensors: dict, num_layers: int, *, head_quant: bool = False, weight_dtype: str = "bf16",
                        tie_word_embeddings: bool = False) -> DecoderWeights:
    """Hugging Face Llama tensors (name -> f32 array, projections [out, in]) -> DecoderWeights with every layer
    projection quantized.  The embedding and an unquantized head keep the model's weight dtype (bf16 values by
    default; WeightQuant.kt:21-22: the head is quantized only under headQuant)."""
    keep = (lambda a: snap_bf16(a)) if weight_dtype == "bf16" else (lambda a: np.ascontiguousarray(a, np.float32))
    w = DecoderWeights(embed=keep(tensors["model.embed_tokens.weight"]))
    for l in range(num_layers):
        pre = f"model.layers.{l}."
        lw = {k: quantize_int8(tensors[pre + hf + ".weight"]) for k, hf in _HF.items()}
        lw["ln1"] = np.ascontiguousarray(tensors[pre + "input_layernorm.weight"], np.float32)
        lw["ln2"] = np.ascontiguousarray(tensors[pre + "post_attention_layernorm.weight"], np.float32)
        w.layers.append(lw)
    w.final_norm = np.ascontiguousarray(tensors["model.norm.weight"], np.float32)
    head = tensors["model.embed_tokens.weight"] if tie_word_embeddings else tensors["lm_head.weight"]
    w.head = quantize_int8(head) if head_quant else keep(np.ascontiguousarray(np.asarray(head, np.float32).T))
    return w


# ---------------------------------------------------------------------------------------------- staged weight files

@dataclass
class StagedFile:
    name: str
    path: str
    dtype: str
    dims: list
    byte_length: int
    sha256: str


class StagedWeights:
    """The staged weight files of an exported model version directory (the one holding tlaloc-serving.json)."""

    def __init__(self, version_dir: str):
        self.dir = version_dir
        with open(os.path.join(version_dir, MANIFEST)) as f:
            self.manifest = json.load(f)
        ptr = self.manifest.get("weights") or {}
        if ptr.get("embedded") or ptr.get("format") != STAGED_FORMAT:
            raise ValueError(f"{version_dir}: weights are {ptr.get('format')!r}; only the 'staged' format (one raw file per "
                             "slot) can be loaded")
        self.files: dict[str, StagedFile] = {}
        for e in ptr.get("table", []):
            f = StagedFile(e["name"], e["path"], e["dtype"], [int(d) for d in e["dims"]], int(e["byteLength"]), e["sha256"])
            if f.name in self.files:
                raise ValueError(f"{version_dir}: duplicate weight slot {f.name!r}")
            if f.dtype not in _DTYPES:
                raise ValueError(f"{version_dir}: slot {f.name!r} has dtype {f.dtype!r}, which this loader does not read")
            want = int(np.prod(f.dims, dtype=np.int64)) * np.dtype(_DTYPES[f.dtype]).itemsize
            if want != f.byte_length:
                raise ValueError(f"{version_dir}: slot {f.name!r} is {f.dtype} {f.dims} = {want} bytes but states {f.byte_length}")
            self.files[f.name] = f

    @property
    def model(self) -> dict:
        return self.manifest.get("model", {})

    def read(self, name: str) -> np.ndarray:
        """A slot's array in its stored dtype (bf16 as uint16 bit patterns)."""
        f = self.files[name]
        path = os.path.join(self.dir, f.path)
        if os.path.getsize(path) != f.byte_length:
            raise ValueError(f"{path}: {os.path.getsize(path)} bytes on disk, the manifest states {f.byte_length}")
        return np.fromfile(path, dtype=np.dtype(_DTYPES[f.dtype]).newbyteorder("<")).reshape(f.dims)

    def read_f32(self, name: str) -> np.ndarray:
        a = self.read(name)
        return bf16_to_f32(a) if self.files[name].dtype == "bf16" else a.astype(np.float32)

    def verify(self) -> list[str]:
        """Slots whose file no longer has the manifest's sha256 (checked on demand, as the reference's loader does)."""
        bad = []
        for f in self.files.values():
            h = hashlib.sha256()
            with open(os.path.join(self.dir, f.path), "rb") as fh:
                for chunk in iter(lambda: fh.read(1 << 24), b""):
                    h.update(chunk)
            if h.hexdigest() != f.sha256:
                bad.append(f.name)
        return bad

    def decoder_weights(self) -> DecoderWeights:
        """The dense Llama-style slots as DecoderWeights: int8 projections keep their codes and scales as staged;
        a projection staged unquantized is refused (this library's projections are int8)."""
        L = int(self.model["numLayers"])

        def proj(slot):
            if self.files[slot].dtype != "i8":
                raise ValueError(f"slot {slot!r} is {self.files[slot].dtype}: this decode path takes int8 projections "
                                 "(export with weightQuant INT8)")
            codes, scales = self.read(slot), self.read(slot + "Scale")
            if scales.shape != (codes.shape[1],):
                raise ValueError(f"slot {slot!r} is {codes.shape} but {slot}Scale is {scales.shape}: scales go with the output axis")
            return np.ascontiguousarray(codes), np.ascontiguousarray(scales, np.float32)

        w = DecoderWeights(embed=self.read_f32("embedTokens"))
        for l in range(L):
            lw = {k: proj(f"{s}{l}") for k, s in _SLOT.items()}
            lw["ln1"] = self.read_f32(f"inputNorm{l}")
            lw["ln2"] = self.read_f32(f"postAttnNorm{l}")
            w.layers.append(lw)
        w.final_norm = self.read_f32("finalNorm")
        w.head = proj("lmHead") if self.files["lmHead"].dtype == "i8" else self.read_f32("lmHead")
        return w


def write_staged(version_dir: str, w: DecoderWeights, model: dict, *, weight_dtype: str = "bf16") -> str:
    """Writes DecoderWeights as the staged files + manifest an exporter leaves (weights section and model shape only:
    the compiled programs of a real artifact are not this library's to write).  Returns the manifest path."""
    wdir = os.path.join(version_dir, STAGED_DIR)
    os.makedirs(wdir, exist_ok=True)
    table = []

    def put(name, arr, tag):
        if tag == "bf16":
            data = f32_to_bf16_bits(arr).astype("<u2")
        else:
            data = np.ascontiguousarray(arr, dtype=np.dtype(_DTYPES[tag]).newbyteorder("<"))
        raw = data.tobytes()
        rel = os.path.join(STAGED_DIR, name + ".bin")
        with open(os.path.join(version_dir, rel), "wb") as f:
            f.write(raw)
        table.append({"name": name, "path": rel, "dtype": tag, "dims": list(arr.shape), "byteLength": len(raw),
                      "sha256": hashlib.sha256(raw).hexdigest()})

    put("embedTokens", w.embed, weight_dtype)
    for l, lw in enumerate(w.layers):
        put(f"inputNorm{l}", lw["ln1"], "f32")
        for k in ("q", "k", "v", "o"):
            put(f"{_SLOT[k]}{l}", lw[k][0], "i8")
            put(f"{_SLOT[k]}{l}Scale", lw[k][1], "f32")
        put(f"postAttnNorm{l}", lw["ln2"], "f32")
        for k in ("gate", "up", "down"):
            put(f"{_SLOT[k]}{l}", lw[k][0], "i8")
            put(f"{_SLOT[k]}{l}Scale", lw[k][1], "f32")
    put("finalNorm", w.final_norm, "f32")
    if isinstance(w.head, tuple):
        put("lmHead", w.head[0], "i8")
        put("lmHeadScale", w.head[1], "f32")
    else:
        put("lmHead", w.head, weight_dtype)
    manifest = {"schemaVersion": "tlaloc-serving-v2", "model": dict(model, numLayers=len(w.layers)),
                "weights": {"format": STAGED_FORMAT, "path": STAGED_DIR, "embedded": False, "table": table}, "entries": []}
    path = os.path.join(version_dir, MANIFEST)
    with open(path, "w") as f:
        json.dump(manifest, f, indent=1)
    return path


# ---------------------------------------------------------------------------------------------- safetensors

def read_safetensors(path: str) -> dict:
    """name -> f32 array of a .safetensors file (F32, BF16 and F16 tensors; 8-byte little-endian header length, a JSON
    header of dtype / shape / data_offsets, then the raw little-endian data)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
        out = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            lo, hi = meta["data_offsets"]
            f.seek(base + lo)
            raw = f.read(hi - lo)
            dt = meta["dtype"]
            if dt == "F32":
                a = np.frombuffer(raw, dtype="<f4").astype(np.float32)
            elif dt == "BF16":
                a = bf16_to_f32(np.frombuffer(raw, dtype="<u2"))
            elif dt == "F16":
                a = np.frombuffer(raw, dtype="<f2").astype(np.float32)
            else:
                raise ValueError(f"{path}: tensor {name!r} has dtype {dt}, which this reader does not widen")
            out[name] = a.reshape(meta["shape"])
    return out
