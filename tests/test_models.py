"""Dense Qwen2 model against the Hugging Face implementation, and checkpoint naming parity
(the reference checks the same with scripts/verify_qwen2_checkpoint.py)."""
import pytest
import torch

from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig


def hf_pair(tied):
    transformers = pytest.importorskip("transformers")
    cfg = Qwen2ModelConfig(vocab_size=160, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=tied)
    hf_cfg = transformers.Qwen2Config(
        vocab_size=160, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=tied,
        rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta, max_position_embeddings=128,
        attention_dropout=0.0, use_sliding_window=False)
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(11)
    hf = transformers.Qwen2ForCausalLM(hf_cfg).eval()
    ours = Qwen2CausalLM(cfg).eval()
    return hf, ours


@pytest.mark.parametrize("tied", [True, False])
def test_logits_and_loss_match_hugging_face_qwen2(tied):
    hf, ours = hf_pair(tied)
    state = {k: v for k, v in hf.state_dict().items()}
    if tied:
        state.pop("lm_head.weight", None)
    missing, unexpected = ours.load_state_dict(state, strict=False)
    assert not unexpected and set(missing) <= {"lm_head.weight"}
    ids = torch.randint(0, 160, (2, 24), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        want = hf(input_ids=ids, labels=ids)
        got = ours(ids, labels=ids)
    torch.testing.assert_close(got.logits, want.logits, atol=2e-5, rtol=2e-5)
    assert got.loss.item() == pytest.approx(want.loss.item(), rel=1e-5)


def test_parameter_names_are_the_hugging_face_names():
    hf, ours = hf_pair(False)
    assert {n for n, _ in ours.named_parameters()} == {n for n, _ in hf.named_parameters()}
    assert all(tuple(p.shape) == tuple(dict(hf.named_parameters())[n].shape)
               for n, p in ours.named_parameters())
