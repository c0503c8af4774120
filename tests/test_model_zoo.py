"""Model families against the Hugging Face implementations: a tiny random model of each family is exported to
safetensors with HF names, loaded by ``transformers`` and both sides must give the same next-token log-probs."""
import pytest
import torch

from siirl_b200.models.config import DecoderConfig, get_config
from siirl_b200.models.decoder import build_model
from siirl_b200.models.hf_io import load_hf_weights, save_hf_model
from siirl_b200.ops.attention import SeqInfo

transformers = pytest.importorskip("transformers")


def _logprobs_ours(model, ids):
    info = SeqInfo([ids.numel()])
    logits = model.logits(ids, info.positions, info)
    return torch.log_softmax(logits.float(), -1)


@pytest.mark.parametrize("preset", ["tiny", "tiny-mixtral", "tiny-qwen2-moe", "tiny-moe"])
def test_family_matches_transformers(preset, tmp_path):
    cfg = get_config(preset)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=4)
    save_hf_model(model, str(tmp_path))
    try:
        hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), torch_dtype=torch.float32,
                                                               attn_implementation="eager")
    except Exception as e:  # noqa: BLE001  (an architecture this transformers build does not ship)
        pytest.skip(f"transformers cannot build {cfg.model_type}: {type(e).__name__}: {e}")
    hf.eval()
    ids = torch.randint(3, cfg.vocab_size, (23,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = torch.log_softmax(hf(ids[None]).logits[0].float(), -1)
        got = _logprobs_ours(model, ids)
    assert (got - want).abs().max().item() < 2e-4, (got - want).abs().max().item()
    # and back: a model filled from the exported files reproduces the original
    cfg2 = DecoderConfig.from_pretrained(str(tmp_path))
    assert cfg2.num_experts == cfg.num_experts and cfg2.norm_topk_prob == cfg.norm_topk_prob
    assert cfg2.shared_expert_intermediate_size == cfg.shared_expert_intermediate_size
    again = build_model(cfg2, dtype=torch.float32, device="cpu", seed=99)
    load_hf_weights(again, str(tmp_path))
    with torch.no_grad():
        assert torch.allclose(_logprobs_ours(again, ids), got, atol=1e-5)
