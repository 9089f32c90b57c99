"""Writing checkpoints the loader reads: a .safetensors file with the reference's tensor names
(design-tests/nn/gpu/src/model.rs:805-918) and the arch.txt line beside it (design-tests/nn/gpu/src/ckpt.rs:115-124).
Reading is the library's job (`ava_ckpt_open`, `ava_b200.engine.Checkpoint`)."""
from __future__ import annotations

import json
import os
import struct

import numpy as np

_DTYPES = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16"}


def dequantised(weights: dict) -> dict:
    """A synthetic model (`ava_b200.synth.model`: int8 matrices with scales) as the f32 tensors a training run would
    have saved: W = q * scale.  Quantising these again per output column gives q and scale back exactly when some
    |q| in every column is 127."""
    out = {}
    for name, w in weights.items():
        if name == "token_bytes":   # the tokenizer's, not the model file's
            continue
        if isinstance(w, tuple):
            q, sc = w
            out[name] = (q.astype(np.float32) * np.asarray(sc, np.float32)[None, :]).astype(np.float32)
        else:
            out[name] = np.asarray(w, np.float32)
    return out


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """tensors: name -> f32 or f16 array.  Layout: u64 header length, JSON header, data; tensors in name order."""
    header, chunks, at = {}, [], 0
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name])
        if a.dtype not in _DTYPES:
            a = a.astype(np.float32)
        raw = a.tobytes()
        header[name] = {"dtype": _DTYPES[a.dtype], "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        chunks.append(raw)
        at += len(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)     # the data starts on an 8-byte boundary
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for c in chunks:
            f.write(c)


def flags_of(cfg: dict) -> str:
    """The arch.txt line of a block-options configuration (kind D), in the reference's flag words."""
    if not cfg["fast_mem"]:
        return ""
    f = [f"--head-size {cfg['head_size']}", "--gates channel"]
    if cfg["value_residual"]:
        f.append("--value-residual")
    f.append(f"--kwta 1/{cfg['hidden'] // cfg['kwta_k']}")
    f.append("--mlp-act " + ("relu2" if cfg["relu2"] else "relu"))
    if cfg["mem_momentum"] > 0:
        f.append(f"--mem-momentum {cfg['mem_momentum']}")
    f.append("--residual " + ("dense" if cfg["dense"] else "plain"))
    if cfg["lif_scale"]:
        f.append("--lif-scale")
    f.append("--spikes " + ("binary", "ternary", "int2")[cfg["spikes"]])
    if cfg["alif"]:
        f.append("--alif")
    if cfg["theta"]:
        f.append("--homeostasis 0.1")
    if cfg.get("stp"):
        f.append("--stp")
    if cfg.get("dendrite"):
        f.append("--dendrite")
    if cfg.get("neuromod"):
        f.append(f"--neuromod {cfg['neuromod']}")
    if cfg.get("thalamus"):
        f.append("--thalamus")
    if cfg.get("cb_units"):
        f.append(f"--cerebellum-head {cfg['cb_units']}")
    if cfg.get("rhythm"):
        f.append("--rhythm")
    if cfg.get("letters"):
        f.append("--letters")
    if cfg.get("dopamine"):
        f.append("--dopamine")
    if cfg.get("mood"):
        f.append("--mood" if cfg["mood"] == 4 else f"--mood-units {cfg['mood']}")
    return " ".join(f)


def save(folder: str, cfg: dict, weights: dict, name: str = "model.safetensors") -> str:
    """A model folder as the reference's tools leave it: NAME.safetensors and, for block options, arch.txt."""
    os.makedirs(folder, exist_ok=True)
    path = os.path.join(folder, name)
    write_safetensors(path, dequantised(weights))
    fl = flags_of(cfg)
    if fl:
        with open(os.path.join(folder, "arch.txt"), "w") as f:
            f.write(fl + "\n")
    return path
