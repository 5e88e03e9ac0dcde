"""Logits of this framework's GPT against Hugging Face implementations of the same architecture, with
the weights moved over by ``tools/convert_hf_checkpoint`` (tiny random models, fp32, CPU)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from keys_values_b200.models.model import GPT  # noqa: E402
from keys_values_b200.tools.convert_hf_checkpoint import config_from_hf, convert_state_dict  # noqa: E402


def _check(hf_model, hf_cfg, atol=2e-4):
    cfg = config_from_hf(hf_cfg.to_dict())
    model = GPT(cfg)
    sd = convert_state_dict(hf_model.state_dict(), cfg)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all("lora" in k for k in missing), missing
    model.eval()
    hf_model.eval()
    ids = torch.randint(0, hf_cfg.vocab_size, (2, 37))
    with torch.no_grad():
        want = hf_model(ids).logits
        got = model(ids)
    torch.testing.assert_close(got, want, atol=atol, rtol=1e-3)


def test_llama_parity():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    hf_cfg = LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0,
                         tie_word_embeddings=False, attn_implementation="eager")
    _check(LlamaForCausalLM(hf_cfg), hf_cfg)


def test_qwen3_parity_with_qk_norm_and_wide_heads():
    from transformers import Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(0)
    hf_cfg = Qwen3Config(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=128, rms_norm_eps=1e-6,
                         rope_theta=1000000.0, tie_word_embeddings=False, attn_implementation="eager")
    _check(Qwen3ForCausalLM(hf_cfg), hf_cfg)


def test_qwen2_parity_with_attention_bias_and_tied_embeddings():
    from transformers import Qwen2Config, Qwen2ForCausalLM

    torch.manual_seed(0)
    hf_cfg = Qwen2Config(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                         tie_word_embeddings=True, attn_implementation="eager")
    _check(Qwen2ForCausalLM(hf_cfg), hf_cfg)


def test_gemma2_parity_with_softcapping_sliding_window_and_post_norms():
    from transformers import Gemma2Config, Gemma2ForCausalLM

    torch.manual_seed(0)
    hf_cfg = Gemma2Config(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=16, max_position_embeddings=128, rms_norm_eps=1e-6,
                          rope_theta=10000.0, sliding_window=16, query_pre_attn_scalar=16, attn_logit_softcapping=50.0,
                          final_logit_softcapping=30.0, attn_implementation="eager")
    hf = Gemma2ForCausalLM(hf_cfg)
    for n, p in hf.named_parameters():  # HF initialises the norm weights to zero (unit offset): make them count
        if "norm" in n:
            torch.nn.init.normal_(p, 0.0, 0.1)
    _check(hf, hf_cfg, atol=5e-4)
