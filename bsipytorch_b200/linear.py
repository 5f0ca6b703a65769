"""Layer replacement: ``BSIQuantizedLinear`` and ``quantize_model_bsi``.

Mirrors ``bsi_ops/benchmarks/verify_accuracy_bsi.py:46-215`` (the layer) and ``:444-486`` (the model
walk) of the reference: same constructor arguments, attributes and counters, same arithmetic
(keys built once from the float32 weight; per forward: quantise+pack the activations, BSI dot,
cast to the activation dtype, add the bias). ``fused=True`` (default) issues the forward as one
extension call; ``fused=False`` goes through the same two entry points the reference layer calls.
"""
from __future__ import annotations

import os
import time
from typing import Dict, Union

import torch
from torch import nn


def _ops():
    import bsipytorch_b200
    return bsipytorch_b200.bsi_ops


class BSIQuantizedLinear(nn.Module):
    """BSI linear layer using prebuilt keys (reference: verify_accuracy_bsi.py:46-215)."""

    def __init__(self, original_linear, decimalPlaces=2, compress_threshold=0.2, query_threshold=None,
                 prefer_cuda: bool = True, fused: bool = True, keep_dense_weight: bool = False):
        super().__init__()
        self.decimalPlaces = int(decimalPlaces)
        self.compress_threshold = float(compress_threshold)
        self.query_compress_threshold = float(query_threshold) if query_threshold is not None else float(compress_threshold)
        self.in_features = original_linear.in_features
        self.out_features = original_linear.out_features
        self.fused = bool(fused)

        if not (prefer_cuda and torch.cuda.is_available()):
            raise RuntimeError("CUDA path required: there is no CPU fallback for BSIQuantizedLinear")

        dense_weight = original_linear.weight.detach().to(torch.float32)
        self.weight_fp32 = dense_weight.cpu() if keep_dense_weight else None
        self.weight_dense_memory_bytes = dense_weight.numel() * dense_weight.element_size()
        if original_linear.bias is not None:
            bias = original_linear.bias.detach().to(torch.float32)
            self.register_buffer("bias", bias)
            self.bias_fp32 = bias.cpu() if keep_dense_weight else None
            self.bias_memory_bytes = bias.numel() * bias.element_size()
        else:
            self.register_buffer("bias", None)
            self.bias_fp32 = None
            self.bias_memory_bytes = 0

        with torch.no_grad():
            # The reference hands the builder a CPU tensor (verify_accuracy_bsi.py:82); a CUDA
            # tensor gives the same integers and skips the host round trip.
            self._bsi_keys_cuda, total_mem_bytes, num_keys, d, _W = _ops().build_bsi_keys_cuda(
                dense_weight, self.decimalPlaces, float(self.compress_threshold))
        assert num_keys == self.out_features and d == self.in_features
        self.weight_bsi_memory_bytes = int(total_mem_bytes)
        self.total_bsi_static_bytes = self.weight_bsi_memory_bytes + self.bias_memory_bytes
        self.verbose = False
        self.collect_stats = False
        self._reset_counters()

    def _reset_counters(self):
        self.dot_ns_total = 0
        self.dot_calls = 0
        self.dot_kernel_ns_per_query_last = 0.0
        self.dot_kernel_ns_per_scalar_last = 0.0
        self.dot_query_vectors_total = 0
        self.dot_output_elements_total = 0
        self.build_ns_total = 0
        self.build_quantize_ns_total = 0
        self.build_pack_ns_total = 0
        self.build_kernel_ns_total = 0
        self.build_calls = 0

    def forward(self, x):
        original_dtype = x.dtype
        original_shape = x.shape
        if x.dim() > 2:
            x = x.reshape(-1, x.shape[-1])
        if os.getenv("BSI_QUERY_FP32", "0") != "0":
            x = x.to(torch.float32)
        ops = _ops()
        batch_inputs = x.detach().contiguous()
        q_rows = int(batch_inputs.shape[0])

        if self.fused and os.getenv("BSI_PROFILE", "0") == "0":
            out = ops.bsi_linear_forward(batch_inputs, self._bsi_keys_cuda, self.bias, self.decimalPlaces)
            if out.dtype != original_dtype:
                out = out.to(original_dtype)
            self.build_calls += 1
            self.dot_calls += 1
        else:
            t0 = time.perf_counter_ns()
            use_packed = os.getenv("BSI_QUERY_PACKED", "1") != "0"
            if use_packed:
                caps = ops.build_bsi_queries_cuda_batch_packed(batch_inputs, self.decimalPlaces,
                                                               float(self.query_compress_threshold))
            else:
                caps = ops.build_bsi_queries_cuda_batch(batch_inputs, self.decimalPlaces,
                                                        float(self.query_compress_threshold))
            self.build_ns_total += time.perf_counter_ns() - t0
            q_ns, p_ns, t_ns = ops.get_last_query_build_profile_cuda()
            self.build_quantize_ns_total += int(q_ns)
            self.build_pack_ns_total += int(p_ns)
            self.build_kernel_ns_total += int(t_ns)
            self.build_calls += 1
            if use_packed:
                scores, ns_total, ns_q, ns_s = ops.batch_dot_product_multiquery_cuda_batch_caps(caps, self._bsi_keys_cuda)
            else:
                scores, ns_total, ns_q, ns_s = ops.batch_dot_product_multiquery_cuda_caps(caps, self._bsi_keys_cuda)
            self.dot_ns_total += int(ns_total)
            self.dot_kernel_ns_per_query_last = float(ns_q)
            self.dot_kernel_ns_per_scalar_last = float(ns_s)
            self.dot_calls += 1
            out = scores.to(dtype=original_dtype)
            if self.bias is not None:
                out = out + self.bias.to(dtype=original_dtype)
        self.dot_query_vectors_total += q_rows
        self.dot_output_elements_total += q_rows * int(self.out_features)
        if len(original_shape) == 3:
            out = out.view(original_shape[0], original_shape[1], -1)
        return out


def reset_bsi_dot_counters(model: nn.Module):
    for m in model.modules():
        if isinstance(m, BSIQuantizedLinear):
            m._reset_counters()


def sum_bsi_dot_counters(model: nn.Module) -> int:
    return sum(int(m.dot_ns_total) for m in model.modules() if isinstance(m, BSIQuantizedLinear))


def bsi_full_model_static_bytes(model: nn.Module) -> int:
    """BSI key bytes + bias bytes over all replaced layers (verify_accuracy_bsi.py:281-300)."""
    return sum(int(m.total_bsi_static_bytes) for m in model.modules() if isinstance(m, BSIQuantizedLinear))


def _resolve_layer_value(config: Union[float, Dict[str, float]], layer_kind: str, fallback: float) -> float:
    if isinstance(config, dict):
        if layer_kind in ("attention", "mlp"):
            return float(config.get(layer_kind, config.get("default", fallback)))
        return float(config.get("default", fallback))
    return float(config)


def quantize_model_bsi(model, decimalPlaces=2, skip_lm_head=True, scope="all", compress_threshold=0.2,
                       prefer_cuda: bool = True, layer_factory=None, verbose: bool = True):
    """Replace ``nn.Linear`` modules by BSI layers (reference: verify_accuracy_bsi.py:444-486).

    scope: 'all' (every Linear except lm_head), 'attention' (q/k/v/out projections) or 'mlp' (fc1/fc2).
    ``layer_factory(linear, decimalPlaces=..., compress_threshold=..., name=...)`` lets the caller build a
    different layer (e.g. an R-sharded one); default ``BSIQuantizedLinear``.
    """
    def is_attention_linear(name: str) -> bool:
        return any(t in name for t in ["attn", "self_attn", "q_proj", "k_proj", "v_proj", "out_proj"])

    def is_mlp_linear(name: str) -> bool:
        return any(t in name for t in ["mlp", "ff", "ffn", "fc1", "fc2"])

    default_decimal = float(decimalPlaces if isinstance(decimalPlaces, (int, float)) else decimalPlaces.get("default", 2))
    default_threshold = float(compress_threshold if isinstance(compress_threshold, (int, float))
                              else compress_threshold.get("default", 0.2))
    targets = []
    for name, module in model.named_modules():
        if isinstance(module, nn.Linear):
            if skip_lm_head and "lm_head" in name:
                continue
            if scope == "attention" and not is_attention_linear(name):
                continue
            if scope == "mlp" and not is_mlp_linear(name):
                continue
            targets.append((name, module))
    for name, module in targets:
        parent = model
        parts = name.split(".")
        for part in parts[:-1]:
            parent = getattr(parent, part)
        kind = "attention" if is_attention_linear(name) else "mlp" if is_mlp_linear(name) else "other"
        dp = _resolve_layer_value(decimalPlaces, kind, default_decimal)
        thr = _resolve_layer_value(compress_threshold, kind, default_threshold)
        if layer_factory is None:
            new = BSIQuantizedLinear(module, decimalPlaces=dp, compress_threshold=thr, prefer_cuda=prefer_cuda)
        else:
            new = layer_factory(module, decimalPlaces=dp, compress_threshold=thr, name=name)
        setattr(parent, parts[-1], new)
    if verbose:
        print(f"Quantized {len(targets)} linear layers to BSI with decimalPlaces={decimalPlaces} (scope={scope})")
    return model
