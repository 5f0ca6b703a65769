"""OPT decoder (random init) whose linear layers run as BSI ops.

The reference evaluates `facebook/opt-*` checkpoints from the HuggingFace hub with every
`nn.Linear` except `lm_head` swapped for `BSIQuantizedLinear`
(bsi_ops/benchmarks/benchmark_performance_bsi.py, verify_accuracy_bsi.py:444-486). There is no
network here, so the architecture is restated (pre-LN decoder, learned positions with offset 2,
ReLU MLP, tied lm_head) and initialised randomly; the module and parameter names follow the
HuggingFace OPT implementation so that `quantize_model_bsi`'s name-based scope selection
(q_proj / k_proj / v_proj / out_proj / fc1 / fc2) works unchanged and a HuggingFace state dict
loads as is. Attention, LayerNorm, embeddings and `lm_head` stay plain torch ops, exactly as in
the reference.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class OPTConfig:
    vocab_size: int = 50272
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    ffn_dim: int = 3072
    max_position_embeddings: int = 2048
    init_std: float = 0.02
    name: str = "opt-125m"


CONFIGS = {
    "opt-125m": OPTConfig(),
    "opt-1.3b": OPTConfig(hidden_size=2048, num_hidden_layers=24, num_attention_heads=32, ffn_dim=8192, name="opt-1.3b"),
    "opt-6.7b": OPTConfig(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, ffn_dim=16384, name="opt-6.7b"),
}


class OPTLearnedPositionalEmbedding(nn.Embedding):
    """Positions are offset by 2 (a quirk of the original OPT checkpoints kept by HuggingFace)."""

    def __init__(self, num_embeddings: int, embedding_dim: int):
        self.offset = 2
        super().__init__(num_embeddings + self.offset, embedding_dim)

    def forward(self, seq_len: int, device):
        pos = torch.arange(seq_len, device=device) + self.offset
        return super().forward(pos)


class OPTAttention(nn.Module):
    def __init__(self, cfg: OPTConfig):
        super().__init__()
        self.num_heads = cfg.num_attention_heads
        self.head_dim = cfg.hidden_size // cfg.num_attention_heads
        h = cfg.hidden_size
        self.k_proj = nn.Linear(h, h)
        self.v_proj = nn.Linear(h, h)
        self.q_proj = nn.Linear(h, h)
        self.out_proj = nn.Linear(h, h)

    def forward(self, x):
        B, T, H = x.shape
        # HuggingFace's OPT scales the query projection by head_dim^-0.5 in the model's type and runs attention
        # with unit scaling ("original order of scaling", modeling_opt.py): for head_dim 128 the factor is not a
        # power of two, so the order matters for bit-identity with the reference's flow
        q = (self.q_proj(x) * self.head_dim ** -0.5).view(B, T, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(B, T, self.num_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(B, T, self.num_heads, self.head_dim).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0)
        return self.out_proj(y.transpose(1, 2).reshape(B, T, H))


class OPTDecoderLayer(nn.Module):
    def __init__(self, cfg: OPTConfig):
        super().__init__()
        self.self_attn = OPTAttention(cfg)
        self.self_attn_layer_norm = nn.LayerNorm(cfg.hidden_size)
        self.fc1 = nn.Linear(cfg.hidden_size, cfg.ffn_dim)
        self.fc2 = nn.Linear(cfg.ffn_dim, cfg.hidden_size)
        self.final_layer_norm = nn.LayerNorm(cfg.hidden_size)

    def forward(self, x):
        x = x + self.self_attn(self.self_attn_layer_norm(x))
        return x + self.fc2(F.relu(self.fc1(self.final_layer_norm(x))))


class OPTDecoder(nn.Module):
    def __init__(self, cfg: OPTConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, padding_idx=1)
        self.embed_positions = OPTLearnedPositionalEmbedding(cfg.max_position_embeddings, cfg.hidden_size)
        self.final_layer_norm = nn.LayerNorm(cfg.hidden_size)
        self.layers = nn.ModuleList([OPTDecoderLayer(cfg) for _ in range(cfg.num_hidden_layers)])

    def forward(self, input_ids):
        x = self.embed_tokens(input_ids) + self.embed_positions(input_ids.shape[1], input_ids.device)
        for layer in self.layers:
            x = layer(x)
        return self.final_layer_norm(x)


class OPTModel(nn.Module):
    def __init__(self, cfg: OPTConfig):
        super().__init__()
        self.decoder = OPTDecoder(cfg)


class OPTForCausalLM(nn.Module):
    """`model.decoder...` / `lm_head` naming as in HuggingFace's OPTForCausalLM."""

    def __init__(self, cfg: OPTConfig):
        super().__init__()
        self.config = cfg
        self.model = OPTModel(cfg)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.lm_head.weight = self.model.decoder.embed_tokens.weight  # tied

    def forward(self, input_ids):
        return self.lm_head(self.model.decoder(input_ids))

    @torch.no_grad()
    def next_token(self, input_ids):
        """Last-position argmax, the reference's accuracy statistic (benchmark_performance_bsi.py:209-212)."""
        hidden = self.model.decoder(input_ids)[:, -1, :]
        return self.lm_head(hidden).argmax(dim=-1)


@torch.no_grad()
def init_weights_(model: OPTForCausalLM, seed: int = 0):
    """HuggingFace's OPT init: normal(0, init_std) for Linear and Embedding weights, zero biases,
    unit LayerNorm. One generator per parameter (seeded by name order) so that every rank of a
    sharded run draws the same values whatever it keeps afterwards."""
    std = model.config.init_std
    for i, (name, p) in enumerate(sorted(model.named_parameters())):
        if name.endswith("layer_norm.weight"):
            p.fill_(1.0)
        elif name.endswith("bias"):
            p.zero_()
        else:
            g = torch.Generator(device=p.device).manual_seed(seed * 1000003 + i)
            p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=g))
    pad = model.model.decoder.embed_tokens.padding_idx
    if pad is not None:
        model.model.decoder.embed_tokens.weight[pad].zero_()
    return model


def build_opt(name: str = "opt-125m", dtype=torch.float32, device="cuda", seed: int = 0) -> OPTForCausalLM:
    cfg = CONFIGS[name] if isinstance(name, str) else name
    with torch.device(device):
        model = OPTForCausalLM(cfg)
    init_weights_(model, seed)
    return model.to(dtype).eval()


@torch.no_grad()
def build_opt_bsi(name: str = "opt-125m", dtype=torch.float16, device="cuda", seed: int = 0, decimal_places: int = 2,
                  compress_threshold: float = 0.5, rank: int = 0, world: int = 1, group=None, keep_dense: bool = False):
    """Random-init OPT with BSI linears, built layer by layer so that the dense weights of a large
    model never sit in memory all at once. world > 1 shards every BSI linear along its output rows."""
    from .linear import BSIQuantizedLinear
    from .sharded import BSIShardedLinear

    cfg = CONFIGS[name] if isinstance(name, str) else name
    std = cfg.init_std
    with torch.device("meta"):
        model = OPTForCausalLM(cfg)
    dec = model.model.decoder
    names = sorted(n for n, _ in model.named_parameters())
    index = {n: i for i, n in enumerate(names)}

    def draw(pname, shape):
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + index[pname])
        return torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=g)

    def materialize_plain(module, prefix):
        for pname, p in list(module.named_parameters(recurse=False)):
            full = prefix + pname
            if full.endswith("layer_norm.weight"):
                val = torch.ones(p.shape, dtype=dtype, device=device)
            elif pname == "bias":
                val = torch.zeros(p.shape, dtype=dtype, device=device)
            else:
                val = draw(full, p.shape).to(dtype)
            setattr(module, pname, nn.Parameter(val, requires_grad=False))

    materialize_plain(dec.embed_tokens, "model.decoder.embed_tokens.")
    if dec.embed_tokens.padding_idx is not None:
        dec.embed_tokens.weight[dec.embed_tokens.padding_idx].zero_()
    materialize_plain(dec.embed_positions, "model.decoder.embed_positions.")
    materialize_plain(dec.final_layer_norm, "model.decoder.final_layer_norm.")
    model.lm_head.weight = dec.embed_tokens.weight
    dense = {}
    for li, layer in enumerate(dec.layers):
        pre = f"model.decoder.layers.{li}."
        materialize_plain(layer.self_attn_layer_norm, pre + "self_attn_layer_norm.")
        materialize_plain(layer.final_layer_norm, pre + "final_layer_norm.")
        for owner, lname, lpre in [(layer.self_attn, "q_proj", pre + "self_attn."), (layer.self_attn, "k_proj", pre + "self_attn."),
                                   (layer.self_attn, "v_proj", pre + "self_attn."), (layer.self_attn, "out_proj", pre + "self_attn."),
                                   (layer, "fc1", pre), (layer, "fc2", pre)]:
            lin_meta = getattr(owner, lname)
            lin = nn.Linear(lin_meta.in_features, lin_meta.out_features, device=device, dtype=torch.float32)
            lin.weight.copy_(draw(lpre + lname + ".weight", lin.weight.shape))
            lin.bias.zero_()
            if keep_dense:
                dense[lpre + lname] = lin.weight.detach().to(dtype).clone()
            if world > 1:
                new = BSIShardedLinear(lin, rank=rank, world=world, group=group, decimalPlaces=decimal_places,
                                       compress_threshold=compress_threshold)
            else:
                new = BSIQuantizedLinear(lin, decimalPlaces=decimal_places, compress_threshold=compress_threshold)
            setattr(owner, lname, new)
            del lin
    model.eval()
    if keep_dense:
        model._dense_weights = dense
    return model
