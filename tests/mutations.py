"""Faults to plant in an engine, one at a time, so that the parity tests can be shown to
catch each of them (the reference's tests do the same to its models: tests/mutation.py:9-22,
tests/parity/test_qwen3.py:98-114 of the reference). A mutation rewrites the model's list of
parts, which is data, and where needed the tensors; nothing in the package is patched."""

from __future__ import annotations

import dataclasses

from mlx_omnia_b200.parts.base import PartSpec
from mlx_omnia_b200.parts.model import LayerSpec, ModelSpec


def _layers(spec: ModelSpec, change) -> ModelSpec:
    """`change(index, block params) -> block params` applied to every layer."""
    layers = tuple(LayerSpec(PartSpec(layer.block.kind, change(i, dict(layer.block.params))), layer.prefix)
                   for i, layer in enumerate(spec.layers))
    return dataclasses.replace(spec, layers=layers)


def _mixer(spec: ModelSpec, **changes) -> ModelSpec:
    def change(_, block):
        mixer = block["mixer"]
        new = {k: (v(mixer.params) if callable(v) else v) for k, v in changes.items()}
        block["mixer"] = PartSpec(mixer.kind, {**mixer.params, **new})
        return block

    return _layers(spec, change)


def _norms(spec: ModelSpec, change) -> ModelSpec:
    """`change(name, norm params) -> norm params` for the block norms of every layer."""
    def per_layer(_, block):
        block["norms"] = {name: PartSpec(norm.kind, change(name, dict(norm.params)))
                          for name, norm in block["norms"].items()}
        return block

    return _layers(spec, per_layer)


def no_plus_one(spec, tensors):
    """The block norms multiply by w instead of 1 + w."""
    return _norms(spec, lambda name, p: {**p, "weight": "plain"}), tensors


def eps_swapped(spec, tensors):
    """The norms before a branch take the eps of the norms after it, and the other way round."""
    pre = spec.layers[0].block.params["norms"]["input_layernorm"].params["eps"]
    post = spec.layers[0].block.params["norms"]["post_attention_layernorm"].params["eps"]
    return _norms(spec, lambda name, p: {**p, "eps": post if p["eps"] == pre else pre}), tensors


def no_gate(spec, tensors):
    """The attention output is not multiplied by the sigmoid gate."""
    return _mixer(spec, gated=False), {k: v for k, v in tensors.items() if "self_attn.gate_proj" not in k}


def nope_rotated(spec, tensors):
    """A layer that is told no positions rotates like its neighbours."""
    dims = spec.layers[0].block.params["mixer"].params["head_dim"]
    return _mixer(spec, position=lambda m: PartSpec("rotary", {"dims": dims, "theta": 1e6})
                  if m["position"].kind == "none" else m["position"]), tensors


def window_plus_one(spec, tensors):
    return _mixer(spec, window=lambda m: None if m["window"] is None else m["window"] + 1), tensors


def window_minus_one(spec, tensors):
    return _mixer(spec, window=lambda m: None if m["window"] is None else m["window"] - 1), tensors


def qk_scale_one(spec, tensors):
    """The softmax scale forgets qk_scale_factor."""
    return _mixer(spec, scale=lambda m: m["head_dim"] ** -0.5), tensors


def no_embedding_norm(spec, tensors):
    return dataclasses.replace(spec, embedding=PartSpec(spec.embedding.kind, {**spec.embedding.params,
                                                                              "norm_eps": None})), tensors


def final_norm_plus_one(spec, tensors):
    """The final norm is treated like the block norms (1 + w)."""
    return dataclasses.replace(spec, final_norm=PartSpec(spec.final_norm.kind, {**spec.final_norm.params,
                                                                                "weight": "centred"})), tensors


def no_qk_norm(spec, tensors):
    return _mixer(spec, qk_norm_eps=None), tensors


def no_softcap(spec, tensors):
    return dataclasses.replace(spec, head=PartSpec(spec.head.kind, {**spec.head.params, "softcap": None})), tensors


ALL = [no_plus_one, eps_swapped, no_gate, nope_rotated, window_plus_one, window_minus_one, qk_scale_one,
       no_embedding_norm, final_norm_plus_one, no_qk_norm, no_softcap]
