"""The restated OPT decoder is the HuggingFace architecture: same parameter names, same logits."""
import pytest
import torch

from bsipytorch_b200 import opt


def test_matches_huggingface_opt_on_a_tiny_config():
    transformers = pytest.importorskip("transformers")
    cfg = opt.OPTConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, ffn_dim=128,
                        max_position_embeddings=64, name="tiny")
    hf_cfg = transformers.OPTConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                    ffn_dim=128, max_position_embeddings=64, word_embed_proj_dim=64,
                                    do_layer_norm_before=True, activation_function="relu", dropout=0.0,
                                    attention_dropout=0.0)
    torch.manual_seed(0)
    hf = transformers.OPTForCausalLM(hf_cfg).eval()
    mine = opt.OPTForCausalLM(cfg).eval()
    missing, unexpected = mine.load_state_dict(hf.state_dict(), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    ids = torch.randint(3, 300, (2, 17))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = mine(ids)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    assert torch.equal(mine.next_token(ids), want[:, -1].argmax(-1))


def test_named_configs_and_init():
    c = opt.CONFIGS["opt-6.7b"]
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.ffn_dim, c.vocab_size) == (4096, 32, 32, 16384, 50272)
    c = opt.CONFIGS["opt-125m"]
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.ffn_dim) == (768, 12, 12, 3072)
    tiny = opt.OPTConfig(vocab_size=100, hidden_size=32, num_hidden_layers=1, num_attention_heads=2, ffn_dim=64,
                         max_position_embeddings=16, name="t")
    a = opt.build_opt(tiny, device="cpu", seed=3)
    b = opt.build_opt(tiny, device="cpu", seed=3)
    c2 = opt.build_opt(tiny, device="cpu", seed=4)
    sa, sb, sc = a.state_dict(), b.state_dict(), c2.state_dict()
    assert all(torch.equal(sa[k], sb[k]) for k in sa)
    assert not torch.equal(sa["model.decoder.layers.0.fc1.weight"], sc["model.decoder.layers.0.fc1.weight"])
    assert abs(float(sa["model.decoder.layers.0.fc1.weight"].std()) - 0.02) < 0.005
    assert a.lm_head.weight is a.model.decoder.embed_tokens.weight
