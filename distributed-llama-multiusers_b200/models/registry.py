"""Which engine serves a model: by the file's kind and, for model directories, by config.json's architecture name.

* ``<file>.m``: the reference's model file (Llama family; header read by formats/mfile.py) -> ``LlamaEngine`` (Q40
  weights), ``F32Engine`` (f32 / f16 weights) or the host backends, chosen in ``cli.app.build_engine``;
* ``<dir>/config.json + model.safetensors``: ``architecture`` names an entry of ``ARCHITECTURES``.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict


def _layer_list(*args, **kw):
    from .layered import LayerListEngine
    return LayerListEngine(*args, **kw)


# architecture name -> engine factory(model_path, rank=, world=, max_rows=, n_slots=, max_seq_len=, dtype=, ...)
ARCHITECTURES: Dict[str, Callable] = {
    "Ribivik": _layer_list,        # mamba2 and latent_attention mixers in the order its configuration lists
    "Sunesun": _layer_list,        # windowed attention (values = keys) + routed experts on hyper-connected residual streams
    "Venadra": _layer_list,        # lightning (linear) attention and chunked sink attention behind a short convolution, PolyNorm / gated experts
    "Darusun": _layer_list,        # post-norm layers: head-mixed grouped-query attention, windowed latent attention with sinks, xIELU / experts with a shared one
}


def is_model_dir(path: str) -> bool:
    return os.path.isdir(path) and os.path.isfile(os.path.join(path, "config.json"))


def architecture_of(model_dir: str) -> str:
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    arch = cfg.get("architecture")
    if not isinstance(arch, str):
        raise ValueError(f"{model_dir}/config.json names no architecture")
    return arch


def engine_for_dir(model_dir: str, **kw):
    """Build the engine of a model directory (GPU only: these models have no host backend)."""
    arch = architecture_of(model_dir)
    if arch not in ARCHITECTURES:
        raise ValueError(f"unknown architecture {arch!r}; known: {', '.join(sorted(ARCHITECTURES))}")
    return ARCHITECTURES[arch](model_dir, **kw)
