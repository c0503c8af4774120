"""Rollout engine on the GPU: paged decode with CUDA graphs equals the eager engine and the full forward."""
import pytest
import torch

from siirl_b200.engine.rollout.native_engine import RolloutEngine, SamplingParams
from siirl_b200.models.config import get_config
from siirl_b200.models.decoder import build_model
from siirl_b200.ops import lib
from siirl_b200.ops.attention import SeqInfo

pytestmark = pytest.mark.gpu


def test_engine_graph_matches_eager_and_forward():
    cfg = get_config("tiny-gpu")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=1)
    prompts = [list(range(5, 5 + n)) for n in (7, 70, 130, 3)]
    sp = SamplingParams(n=2, temperature=0.0, max_new_tokens=20, eos_token_id=None)
    eager = RolloutEngine(model, max_num_seqs=8, max_model_len=512, num_blocks=64, use_cuda_graph=False,
                          sync_interval=4).generate(prompts, sp)
    graph = RolloutEngine(model, max_num_seqs=8, max_model_len=512, num_blocks=64, use_cuda_graph=True,
                          sync_interval=4).generate(prompts, sp)
    lib.check_status()
    assert [o.token_ids for o in eager] == [o.token_ids for o in graph]
    # teacher-forced check: the engine's log-probs agree with a full forward over prompt + response
    for o in graph:
        ids = prompts[o.prompt_index] + o.token_ids
        info = SeqInfo([len(ids)], device="cuda")
        t = torch.tensor(ids, device="cuda")
        lp, _ = model.logprobs(t, info.positions, info, torch.roll(t, -1), with_entropy=False)
        P = len(prompts[o.prompt_index])
        want = lp[P - 1: P - 1 + len(o.token_ids)].cpu()
        got = torch.tensor(o.logprobs)
        assert (want - got).abs().max().item() < 0.08


def test_engine_sampling_runs_and_stops_on_eos():
    cfg = get_config("tiny-gpu")
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=2)
    eng = RolloutEngine(model, max_num_seqs=16, max_model_len=256, num_blocks=64, sync_interval=8)
    prompts = [[7, 8, 9, 10]] * 3
    outs = eng.generate(prompts, SamplingParams(n=4, temperature=1.0, max_new_tokens=24, eos_token_id=5, seed=11))
    assert len(outs) == 12
    for o in outs:
        assert 1 <= len(o.token_ids) <= 24
        if o.finish_reason == "stop":
            assert o.token_ids[-1] == 5 and 5 not in o.token_ids[:-1]
    # samples of one prompt differ
    assert len({tuple(o.token_ids) for o in outs if o.prompt_index == 0}) > 1
    assert eng.alloc.num_free == eng.alloc.num_blocks


def test_lora_adapters_forward_backward_on_gpu():
    """LoRA projections (rank-8 GEMMs: N = 8 and K = 8 tiles) against a PyTorch reference of the same module."""
    import torch

    from siirl_b200.models.config import get_config
    from siirl_b200.models.decoder import build_model
    from siirl_b200.ops import lib
    from siirl_b200.ops.attention import SeqInfo
    cfg = get_config("tiny-gpu")
    cfg.lora_rank, cfg.lora_alpha = 8, 16.0
    m = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=1)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("_lora_B"):
                p.normal_(0, 0.05)
    info = SeqInfo([40, 25], device="cuda")
    ids = torch.randint(3, cfg.vocab_size, (65,), device="cuda")
    h_on = m.forward_hidden(ids, info.positions, info)
    m.set_lora_enabled(False)
    h_off = m.forward_hidden(ids, info.positions, info)
    m.set_lora_enabled(True)
    assert (h_on.float() - h_off.float()).abs().max().item() > 1e-3       # the adapters change the output
    # CPU fp32 twin with the same weights
    mc = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    mc.load_state_dict({k: v.float().cpu() for k, v in m.state_dict().items()})
    ic = SeqInfo([40, 25], device="cpu")
    hc = mc.forward_hidden(ids.cpu(), ic.positions, ic)
    assert (h_on.float().cpu() - hc).abs().max().item() < 0.1
    h_on.float().square().mean().backward()
    hc.square().mean().backward()
    ga = m.layers[0].qkv_proj_lora_A.grad.float().cpu()
    gc = mc.layers[0].qkv_proj_lora_A.grad
    assert (ga - gc).abs().max().item() < 0.05 * max(1.0, gc.abs().max().item()) + 1e-3
    torch.cuda.synchronize()
    lib.check_status()
