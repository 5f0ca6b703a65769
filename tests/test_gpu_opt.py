"""OPT decoder with BSI linears (random init, uniform random token ids stand in for LAMBADA)."""
import numpy as np
import pytest
import torch

from bsipytorch_b200 import opt
from bsipytorch_b200.linear import BSIQuantizedLinear, quantize_model_bsi
from oracle import oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda"
TINY = opt.OPTConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, ffn_dim=1024,
                     max_position_embeddings=128, name="tiny")


def test_layer_by_layer_build_equals_quantize_model_walk():
    dense = opt.build_opt(TINY, dtype=torch.float32, device=DEV, seed=5)
    a = opt.build_opt_bsi(TINY, dtype=torch.float32, device=DEV, seed=5)
    b = quantize_model_bsi(opt.build_opt(TINY, dtype=torch.float32, device=DEV, seed=5), decimalPlaces=2,
                           compress_threshold=0.5, verbose=False)
    n = sum(isinstance(m, BSIQuantizedLinear) for m in a.modules())
    assert n == 2 * 6 == sum(isinstance(m, BSIQuantizedLinear) for m in b.modules())
    assert isinstance(b.lm_head, torch.nn.Linear)
    ids = torch.randint(0, 512, (3, 40), generator=torch.Generator().manual_seed(1)).to(DEV)
    with torch.no_grad():
        la, lb, ld = a(ids), b(ids), dense(ids)
    assert torch.equal(la, lb)                       # same keys, same arithmetic
    assert torch.isfinite(la).all()
    # BSI model tracks the dense model (quantisation error only)
    rel = float((la - ld).norm() / ld.norm())
    assert rel < 0.5, rel     # weights ~N(0, 0.02) on a 0.01 grid: the recipe's own quantisation error


def test_first_bsi_layer_matches_cpu_checker_inside_the_model():
    model = opt.build_opt_bsi(TINY, dtype=torch.float32, device=DEV, seed=2, keep_dense=True)
    ids = torch.randint(0, 512, (2, 24), generator=torch.Generator().manual_seed(3)).to(DEV)
    layer0 = model.model.decoder.layers[0]
    captured = {}
    h = layer0.self_attn.q_proj.register_forward_hook(lambda m, i, out: captured.update(x=i[0].detach(), y=out.detach()))
    with torch.no_grad():
        model(ids)
    h.remove()
    x = captured["x"].reshape(-1, 256).cpu().numpy()
    w = model._dense_weights["model.decoder.layers.0.self_attn.q_proj"].float().cpu().numpy()
    want = o.fixed_dot(x, w)                          # bias is zero at init
    got = captured["y"].reshape(-1, 256).cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_opt125m_forward_batch8_seq128(dtype):
    model = opt.build_opt_bsi("opt-125m", dtype=dtype, device=DEV, seed=0)
    ids = torch.randint(0, 50272, (8, 128), generator=torch.Generator().manual_seed(0)).to(DEV)
    with torch.no_grad():
        tok = model.next_token(ids)
        for m in model.modules():
            if isinstance(m, BSIQuantizedLinear):
                m.fused = False                       # the reference's two-call path
        tok_unfused = model.next_token(ids)
    assert tok.shape == (8,) and torch.equal(tok, tok_unfused)
    if dtype == torch.float32:
        dense = opt.build_opt("opt-125m", dtype=torch.float32, device=DEV, seed=0)
        with torch.no_grad():
            ld = dense(ids)[:, -1]
            for m in model.modules():
                if isinstance(m, BSIQuantizedLinear):
                    m.fused = True
            lb = model(ids)[:, -1]
        assert float((lb - ld).norm() / ld.norm()) < 0.6


def test_tensor_parallel_forward_on_one_rank_equals_the_per_linear_model():
    """World size 1 of the tensor-parallel decoder (fused QKV key set, ReLU inside the fc1 epilogue,
    activations packed once per consumer) gives the logits of the BSIQuantizedLinear-per-layer model."""
    from bsipytorch_b200.opt_tp import build_opt_tp

    cfg = opt.OPTConfig(vocab_size=512, hidden_size=512, num_hidden_layers=2, num_attention_heads=8, ffn_dim=2048,
                        max_position_embeddings=128, name="tiny")
    ids = torch.randint(0, 512, (4, 32), generator=torch.Generator().manual_seed(2)).to(DEV)
    for dtype in (torch.float16, torch.float32):
        ref = opt.build_opt_bsi(cfg, dtype=dtype, device=DEV, seed=11)
        tp = build_opt_tp(cfg, dtype=dtype, device=DEV, seed=11)
        with torch.no_grad():
            want, got = ref(ids), tp(ids)
        assert torch.isfinite(got).all()
        assert torch.equal(got, want)
        assert torch.equal(tp.next_token(ids), ref.next_token(ids))
        tp.capture(4, 32)                                   # replayed from a CUDA graph: same values
        assert torch.equal(tp(ids), want)
        ids2 = torch.randint(0, 512, (4, 32), generator=torch.Generator().manual_seed(9)).to(DEV)
        assert torch.equal(tp(ids2), ref(ids2))


def test_linear_from_packed_relu_and_column_block_pack():
    """pack_queries_into writes a column block of a wider int8 matrix; linear_from_packed with relu=True
    equals relu of the plain call."""
    from bsipytorch_b200 import bsi_ops

    g = torch.Generator().manual_seed(4)
    x = torch.randn(96, 1024, generator=g).half().to(DEV)
    w = (torch.randn(320, 1024, generator=g) * 0.02).to(DEV)
    cap = bsi_ops.build_bsi_keys_cuda(w, 2, 0.5)[0]
    q8 = torch.zeros(96, 1024, dtype=torch.int8, device=DEV)
    sc = torch.zeros(96, 4, dtype=torch.float32, device=DEV)
    for c in range(2):   # two 512-wide feature blocks packed separately, as two ranks would
        blk_sc = torch.empty(96, 2, dtype=torch.float32, device=DEV)
        bsi_ops.pack_queries_into(x[:, c * 512:(c + 1) * 512], q8[:, c * 512:(c + 1) * 512], blk_sc, 2)
        sc[:, c * 2:(c + 1) * 2] = blk_sc
    bias = torch.randn(320, generator=g).to(DEV)
    y = bsi_ops.linear_from_packed(q8, sc, cap, bias, 2, torch.float16, False)
    want = bsi_ops.bsi_linear_forward(x, cap, bias, 2)
    assert torch.equal(y, want)
    yr = bsi_ops.linear_from_packed(q8, sc, cap, bias, 2, torch.float16, True)
    assert torch.equal(yr, torch.relu(want))
    assert (want < 0).any()
