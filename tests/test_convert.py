"""The package's Llama and GPT blocks against the Hugging Face implementations of
the same architectures (random weights, CPU, fp32): converted weights must give the
same logits, and converting back must give the original tensors."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from flextrain_b200.models import convert  # noqa: E402
from flextrain_b200.models.gpt import GPTModel  # noqa: E402
from flextrain_b200.models.llama import LlamaModel  # noqa: E402


def _logits(model, tokens):
    if isinstance(model, LlamaModel):
        x, cos, sin = model.pre_process(tokens)
        for blk in model.blocks:
            x = blk(x, cos, sin)
        return model.post_process(x) @ model.lm_head.t()
    x = model.pre_process(tokens)
    for blk in model.blocks:
        x = blk(x)
    head = model.wte if model.lm_head is None else model.lm_head
    return model.post_process(x) @ head.t()


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_llama_matches_hugging_face(kv_heads):
    torch.manual_seed(0)
    hf_cfg = transformers.LlamaConfig(vocab_size=320, hidden_size=128, intermediate_size=344,
                                      num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=kv_heads, max_position_embeddings=64,
                                      rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False,
                                      attention_bias=False, mlp_bias=False)
    hf = transformers.LlamaForCausalLM(hf_cfg).eval()
    cfg = convert.llama_config_from_hf(hf_cfg)
    assert (cfg.num_layers, cfg.hidden, cfg.num_kv_heads, cfg.ffn) == (2, 128, kv_heads, 344)
    mine = LlamaModel(cfg).eval()
    sd = convert.llama_from_hf(hf.state_dict(), cfg)
    assert set(sd) == set(dict(mine.named_parameters()))
    mine.load_state_dict(sd)
    tokens = torch.randint(0, 320, (2, 48))
    with torch.no_grad():
        want = hf(tokens).logits
        got = _logits(mine, tokens)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), float((got - want).abs().max())
    back = convert.llama_to_hf(sd, cfg)
    for name, t in hf.state_dict().items():
        if name in back:
            assert torch.equal(back[name], t), name
    assert {n for n in hf.state_dict() if "rotary" not in n} <= set(back)


def test_gpt2_matches_hugging_face():
    torch.manual_seed(0)
    hf_cfg = transformers.GPT2Config(vocab_size=320, n_positions=64, n_embd=128, n_layer=2, n_head=4,
                                     resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    hf = transformers.GPT2LMHeadModel(hf_cfg).eval()
    # give the biases and gains some content (they start at 0 / 1)
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(0.05 * torch.randn_like(p))
    cfg = convert.gpt2_config_from_hf(hf_cfg)
    assert (cfg.num_layers, cfg.hidden, cfg.ffn, cfg.tie_embeddings) == (2, 128, 512, True)
    mine = GPTModel(cfg).eval()
    sd = convert.gpt2_from_hf(hf.state_dict(), cfg)
    assert set(sd) == set(dict(mine.named_parameters()))
    mine.load_state_dict(sd)
    tokens = torch.randint(0, 320, (2, 48))
    with torch.no_grad():
        want = hf(tokens).logits
        got = _logits(mine, tokens)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), float((got - want).abs().max())
    back = convert.gpt2_to_hf(sd, cfg)
    hf_sd = hf.state_dict()
    for name, t in back.items():
        assert torch.equal(t, hf_sd[name]), name
    with pytest.raises(ValueError):
        convert.gpt2_config_from_hf(transformers.GPT2Config(activation_function="relu"))
