"""BSI linear layer with a single-call forward, and helpers around it.

The reference defines its layer replacement in a benchmark script (``BSIQuantizedLinear`` and
``quantize_model_bsi``, bsi_ops/benchmarks/verify_accuracy_bsi.py:46-215, 444-486). That class runs
unmodified over this package's ``bsi_ops`` module (``install_as_bsi_ops()``; tests/test_gpu_reference_callers.py
does exactly that), so nothing here restates its bookkeeping (timing counters, diagnostics, summaries).
What this module adds:

* a layer whose forward is ONE extension call -- quantise + pack, integer dot, float32 chunk combine,
  cast and bias in the dot's epilogue -- with bit-identical results (``fused=False`` issues the same two
  entry points the reference's layer calls);
* key sets that can be written to and read from disk in their packed form (``save_bsi_keysets`` /
  ``load_bsi_keysets``), so a model is not quantised again on every start;
* a model walk that accepts a layer factory (used for the R-sharded layer).
"""
from __future__ import annotations

import os
from typing import Callable, Dict, Optional, Union

import torch
from torch import nn


def _ops():
    import bsipytorch_b200
    return bsipytorch_b200.bsi_ops


class BSIQuantizedLinear(nn.Module):
    """``y = x @ W.T + b`` on the BSI path. Constructor arguments as the reference's layer
    (verify_accuracy_bsi.py:49); ``keyset`` builds the layer from a stored key set instead of a dense weight."""

    def __init__(self, original_linear: Optional[nn.Linear] = None, decimalPlaces=2, compress_threshold=0.2,
                 query_threshold=None, prefer_cuda: bool = True, fused: bool = True, keyset: Optional[str] = None,
                 bias: Optional[torch.Tensor] = None):
        super().__init__()
        if not (prefer_cuda and torch.cuda.is_available()):
            raise RuntimeError("CUDA path required: there is no CPU fallback for BSIQuantizedLinear")
        self.decimalPlaces = int(decimalPlaces)
        self.compress_threshold = float(compress_threshold)
        self.query_compress_threshold = float(query_threshold) if query_threshold is not None else float(compress_threshold)
        self.fused = bool(fused)
        ops = _ops()
        dev = torch.device("cuda", torch.cuda.current_device())
        if original_linear is not None and original_linear.weight.is_cuda:
            dev = original_linear.weight.device
        with torch.no_grad(), torch.cuda.device(dev):
            if keyset is not None:
                self._bsi_keys_cuda, mem, self.out_features, self.in_features, _w = ops.load_keyset(keyset)
                self.decimalPlaces = int(ops.bsi_keys_cuda_stats(self._bsi_keys_cuda)["decimals"])
            else:
                self.in_features, self.out_features = original_linear.in_features, original_linear.out_features
                # the reference hands the builder a CPU copy (verify_accuracy_bsi.py:82); the tensor as it is gives
                # the same integers without the host round trip
                self._bsi_keys_cuda, mem, num_keys, d, _w = ops.build_bsi_keys_cuda(
                    original_linear.weight.detach().to(torch.float32), self.decimalPlaces, self.compress_threshold)
                assert num_keys == self.out_features and d == self.in_features
                if bias is None and original_linear.bias is not None:
                    bias = original_linear.bias
        self.register_buffer("bias", None if bias is None else bias.detach().to(torch.float32).to(dev))
        self.weight_bsi_memory_bytes = int(mem)
        self.total_bsi_static_bytes = self.weight_bsi_memory_bytes + (0 if self.bias is None else self.bias.numel() * 4)
        self.dot_calls = 0
        self.dot_output_elements_total = 0

    def forward(self, x):
        shape, dtype = x.shape, x.dtype
        x2d = x.reshape(-1, shape[-1]).detach().contiguous()
        if os.getenv("BSI_QUERY_FP32", "0") != "0":          # the reference's switch (verify_accuracy_bsi.py:126)
            x2d = x2d.to(torch.float32)
        ops = _ops()
        if self.fused and os.getenv("BSI_PROFILE", "0") == "0":
            out = ops.bsi_linear_forward(x2d, self._bsi_keys_cuda, self.bias, self.decimalPlaces)
            out = out if out.dtype == dtype else out.to(dtype)
        else:
            packed = os.getenv("BSI_QUERY_PACKED", "1") != "0"
            build = ops.build_bsi_queries_cuda_batch_packed if packed else ops.build_bsi_queries_cuda_batch
            dot = ops.batch_dot_product_multiquery_cuda_batch_caps if packed else ops.batch_dot_product_multiquery_cuda_caps
            scores, *_ = dot(build(x2d, self.decimalPlaces, self.query_compress_threshold), self._bsi_keys_cuda)
            out = scores.to(dtype)
            if self.bias is not None:
                out = out + self.bias.to(dtype)
        self.dot_calls += 1
        self.dot_output_elements_total += x2d.shape[0] * self.out_features
        return out.view(*shape[:-1], self.out_features)


def bsi_layers(model: nn.Module):
    """(name, layer) of every BSI layer of `model` that owns a key set capsule (this class or the reference's)."""
    return [(n, m) for n, m in model.named_modules() if getattr(m, "_bsi_keys_cuda", None) is not None]


def bsi_full_model_static_bytes(model: nn.Module) -> int:
    """Key bytes + bias bytes over all BSI layers."""
    return sum(int(getattr(m, "total_bsi_static_bytes", 0)) for _, m in bsi_layers(model))


def save_bsi_keysets(model: nn.Module, out_dir: str) -> int:
    """Writes the key set of every BSI layer to ``out_dir/<layer name>/keyset.bsik`` (row scales + EWAH / verbatim
    slice streams) and the biases to ``out_dir/biases.pt``; returns the bytes written for the key sets."""
    ops = _ops()
    total, biases = 0, {}
    for name, layer in bsi_layers(model):
        ops.save_keyset(layer._bsi_keys_cuda, os.path.join(out_dir, name))
        total += int(ops.keyset_size_on_disk(layer._bsi_keys_cuda)[1])
        if getattr(layer, "bias", None) is not None:
            biases[name] = layer.bias.detach().float().cpu()
    torch.save(biases, os.path.join(out_dir, "biases.pt"))
    return total


def load_bsi_keysets(model: nn.Module, in_dir: str, fused: bool = True) -> nn.Module:
    """Replaces every ``nn.Linear`` (or BSI layer) of `model` that has a stored key set under `in_dir` by a BSI
    layer built from it: no dense weight is read and nothing is quantised again."""
    biases = torch.load(os.path.join(in_dir, "biases.pt"))
    for name, module in list(model.named_modules()):
        if not os.path.exists(os.path.join(in_dir, name, "keyset.bsik")) or not name:
            continue
        parent = model
        parts = name.split(".")
        for part in parts[:-1]:
            parent = getattr(parent, part)
        setattr(parent, parts[-1], BSIQuantizedLinear(keyset=os.path.join(in_dir, name), bias=biases.get(name), fused=fused))
    return model


def _layer_value(config: Union[float, Dict[str, float]], kind: str, fallback: float) -> float:
    if isinstance(config, dict):
        return float(config.get(kind, config.get("default", fallback)))
    return float(config)


_ATTENTION = ("attn", "self_attn", "q_proj", "k_proj", "v_proj", "out_proj")
_MLP = ("mlp", "ff", "ffn", "fc1", "fc2")


def quantize_model_bsi(model, decimalPlaces=2, skip_lm_head=True, scope="all", compress_threshold=0.2,
                       prefer_cuda: bool = True, layer_factory: Optional[Callable] = None, verbose: bool = True):
    """Swaps ``nn.Linear`` modules for BSI layers, with the selection rules of the reference's walk
    (verify_accuracy_bsi.py:444-486): every Linear except ``lm_head``; ``scope`` 'attention' or 'mlp' narrows it by
    name; ``decimalPlaces`` / ``compress_threshold`` may be dicts keyed by 'attention' / 'mlp' / 'default'.
    ``layer_factory(linear, decimalPlaces=..., compress_threshold=..., name=...)`` builds another layer type."""
    picked = []
    for name, module in model.named_modules():
        if not isinstance(module, nn.Linear) or (skip_lm_head and "lm_head" in name):
            continue
        kind = "attention" if any(t in name for t in _ATTENTION) else "mlp" if any(t in name for t in _MLP) else "other"
        if scope in ("attention", "mlp") and kind != scope:
            continue
        picked.append((name, module, kind))
    for name, module, kind in picked:
        dp = _layer_value(decimalPlaces, kind, 2)
        thr = _layer_value(compress_threshold, kind, 0.2)
        new = (BSIQuantizedLinear(module, decimalPlaces=dp, compress_threshold=thr, prefer_cuda=prefer_cuda)
               if layer_factory is None else layer_factory(module, decimalPlaces=dp, compress_threshold=thr, name=name))
        parent = model
        parts = name.split(".")
        for part in parts[:-1]:
            parent = getattr(parent, part)
        setattr(parent, parts[-1], new)
    if verbose:
        print(f"Quantized {len(picked)} linear layers to BSI with decimalPlaces={decimalPlaces} (scope={scope})")
    return model
