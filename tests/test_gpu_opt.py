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


def test_model_keysets_round_trip_through_disk(tmp_path):
    """save_bsi_keysets / load_bsi_keysets: a model rebuilt from the stored key sets (no dense linear weights read,
    nothing quantised again) gives the logits of the model that wrote them."""
    from bsipytorch_b200.linear import load_bsi_keysets, save_bsi_keysets

    src = opt.build_opt_bsi(TINY, dtype=torch.float16, device=DEV, seed=5)
    with torch.no_grad():
        for i, layer in enumerate(src.model.decoder.layers):     # non-zero biases, so that they are seen to travel
            layer.fc1.bias.copy_(torch.full_like(layer.fc1.bias, 0.01 * (i + 1)))
    written = save_bsi_keysets(src, str(tmp_path))
    assert written > 0
    dst = opt.build_opt(TINY, dtype=torch.float16, device=DEV, seed=5)
    for layer in dst.model.decoder.layers:                       # prove the dense weights are not what is used
        for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.out_proj,
                    layer.fc1, layer.fc2):
            lin.weight.data.zero_()
    load_bsi_keysets(dst, str(tmp_path))
    assert sum(isinstance(m, BSIQuantizedLinear) for m in dst.modules()) == 12
    ids = torch.randint(0, 512, (3, 40), generator=torch.Generator().manual_seed(1)).to(DEV)
    with torch.no_grad():
        assert torch.equal(dst(ids), src(ids))


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
        # every fused piece (QKV key set, ReLU and re-quantisation inside the fc1 epilogue) is exact and LayerNorm is
        # torch's: the logits are those of the per-linear model bit for bit, in every layer type
        assert torch.equal(got, want)
        assert torch.equal(tp.next_token(ids), ref.next_token(ids))
        if dtype == torch.float16:
            # opt-in add + LayerNorm + pack kernel: same formula as torch's LayerNorm, float32 statistics in another
            # summation order; the rare last-bit difference is amplified by the following re-quantisations
            fused = build_opt_tp(cfg, dtype=dtype, device=DEV, seed=11, fuse_ln=True)
            with torch.no_grad():
                gf = fused(ids)
            rel = float((gf.float() - want.float()).norm() / want.float().norm())
            assert torch.isfinite(gf).all() and rel < 5e-2, rel
        tp.capture(4, 32)                                   # replayed from a CUDA graph: same values
        assert torch.equal(tp(ids), got)
        ids2 = torch.randint(0, 512, (4, 32), generator=torch.Generator().manual_seed(9)).to(DEV)
        eager = build_opt_tp(cfg, dtype=dtype, device=DEV, seed=11)
        assert torch.equal(tp(ids2), eager(ids2))


def test_add_layernorm_pack_against_torch():
    from bsipytorch_b200 import bsi_ops

    g = torch.Generator().manual_seed(21)
    for dtype, H, rows in [(torch.float16, 1024, 70), (torch.bfloat16, 768, 33), (torch.float16, 4096, 16)]:
        x = torch.randn(rows, H, generator=g).to(dtype).to(DEV)
        d = (0.3 * torch.randn(rows, H, generator=g)).to(dtype).to(DEV)
        ln = torch.nn.LayerNorm(H, device=DEV, dtype=dtype)
        with torch.no_grad():
            ln.weight.copy_(1.0 + 0.1 * torch.randn(H, generator=g).to(DEV))
            ln.bias.copy_(0.1 * torch.randn(H, generator=g).to(DEV))
        q8 = torch.full((rows, H), 99, dtype=torch.int8, device=DEV)
        sc = torch.full((rows, H // 256), -1.0, device=DEV)
        out = bsi_ops.add_layernorm_pack(x, d, ln.weight, ln.bias, ln.eps, [q8.data_ptr()], H, [sc.data_ptr()], H // 256, 2)
        assert torch.equal(out, x + d)                       # the residual sum is exact
        with torch.no_grad():
            y = ln(x + d)
        want_q8 = torch.empty_like(q8)
        want_sc = torch.empty_like(sc)
        bsi_ops.pack_queries_into(y, want_q8, want_sc, 2)
        # the library's LayerNorm may differ from torch's in the last bit of y: integers within one step, almost all equal
        diff = (q8.int() - want_q8.int()).abs()
        same_scale = (sc == want_sc)
        assert same_scale.float().mean() > 0.98
        mask = same_scale.repeat_interleave(256, dim=1)
        assert int(diff[mask].max()) <= 1 and float((diff[mask] > 0).float().mean()) < 0.02
        # no delta: x passes through untouched
        out2 = bsi_ops.add_layernorm_pack(x, None, ln.weight, ln.bias, ln.eps, [q8.data_ptr()], H, [sc.data_ptr()], H // 256, 2)
        assert out2.data_ptr() == x.data_ptr()
    assert bsi_ops.device_status() == 0


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


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_exact_integer_route_does_not_change_the_model(dtype, monkeypatch):
    """The dots accumulate in integers where a bound proves that exact; with the route switched off the per-linear
    and the tensor-parallel model give the same logits bit for bit, and the route is actually taken when it is on."""
    from bsipytorch_b200 import capi
    from bsipytorch_b200.opt_tp import build_opt_tp
    cfg = opt.OPTConfig(vocab_size=512, hidden_size=512, num_hidden_layers=2, num_attention_heads=8, ffn_dim=2048,
                        max_position_embeddings=128, name="tiny512")
    ids = torch.randint(0, 512, (8, 64), generator=torch.Generator().manual_seed(3)).to(DEV)      # 512 tokens: paired kernel
    per_linear = opt.build_opt_bsi(cfg, dtype=dtype, device=DEV, seed=7)
    tp = build_opt_tp(cfg, dtype=dtype, device=DEV, seed=7)
    capi.exact_int_tiles()
    with torch.no_grad():
        on = per_linear(ids), tp(ids)
    assert capi.exact_int_tiles() > 0
    monkeypatch.setenv("BSI_B200_EXACT_INT", "0")
    with torch.no_grad():
        off = per_linear(ids), tp(ids)
    assert capi.exact_int_tiles() == 0
    assert torch.equal(on[0], off[0]) and torch.equal(on[1], off[1])
