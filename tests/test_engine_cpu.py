"""CPU checks of the model path: packing, decoder, rollout engine, flat parameter store, checkpoints, rewards."""
import os

import pytest
import torch

from siirl_b200.data_coordinator import Batch
from siirl_b200.engine.packing import get_response_mask, pack_batch
from siirl_b200.engine.reward_manager import DAPORewardManager, NaiveRewardManager
from siirl_b200.engine.rollout.native_engine import RolloutEngine, SamplingParams
from siirl_b200.models.config import DecoderConfig, get_config
from siirl_b200.models.decoder import build_model
from siirl_b200.models.hf_io import load_hf_weights, save_hf_model
from siirl_b200.ops.attention import SeqInfo
from siirl_b200.parallel.flat_params import FlatParamStore, lr_at_step
from siirl_b200.params import parse_config
from siirl_b200.data_coordinator.dataloader import SyntheticTokenizer
from siirl_b200.utils.checkpoint.checkpoint_manager import ShardedCheckpointManager


@pytest.fixture(scope="module")
def tiny():
    return build_model(get_config("tiny"), dtype=torch.float32, seed=0)


def test_pack_batch_indices():
    P, R = 4, 3
    ids = torch.tensor([[0, 0, 11, 12, 21, 22, 0], [0, 31, 32, 33, 41, 0, 0]])
    am = torch.tensor([[0, 0, 1, 1, 1, 1, 0], [0, 1, 1, 1, 1, 0, 0]])
    pk = pack_batch(ids, am, R)
    assert pk.input_ids.tolist() == [11, 12, 21, 22, 31, 32, 33, 41]
    assert pk.positions.tolist() == [0, 1, 2, 3, 0, 1, 2, 3]
    assert pk.info.seqlens == [4, 4]
    # position that predicts response token k: last prompt token + k
    assert pk.sel.tolist() == [1, 2, 6] and pk.labels.tolist() == [21, 22, 41]
    out = pk.scatter(torch.tensor([1.0, 2.0, 3.0]))
    assert out.tolist() == [[1.0, 2.0, 0.0], [3.0, 0.0, 0.0]]


def test_response_mask_stops_after_first_eos():
    r = torch.tensor([[5, 2, 7, 2], [5, 6, 7, 8]])
    assert get_response_mask(r, 2).tolist() == [[1, 1, 0, 0], [1, 1, 1, 1]]


def test_packed_forward_equals_per_sequence_forward(tiny):
    ids = torch.randint(3, 1000, (17,))
    info = SeqInfo([6, 11])
    both = tiny.logits(ids, info.positions, info)
    a = tiny.logits(ids[:6], SeqInfo([6]).positions, SeqInfo([6]))
    b = tiny.logits(ids[6:], SeqInfo([11]).positions, SeqInfo([11]))
    torch.testing.assert_close(both, torch.cat([a, b]), rtol=1e-4, atol=1e-4)


def test_engine_matches_naive_greedy_with_prefix_sharing(tiny):
    eng = RolloutEngine(tiny, max_num_seqs=8, max_model_len=256, sync_interval=4)
    prompts = [[5, 6, 7, 8, 9], list(range(20, 20 + 70))]
    outs = eng.generate(prompts, SamplingParams(n=2, temperature=0.0, max_new_tokens=6))
    for o in outs:
        seq = list(prompts[o.prompt_index])
        for _ in range(6):
            info = SeqInfo([len(seq)])
            seq.append(int(tiny.logits(torch.tensor(seq), info.positions, info)[-1].argmax()))
        assert o.token_ids == seq[len(prompts[o.prompt_index]):]
    assert eng.alloc.num_free == eng.alloc.num_blocks
    eng.sleep()
    assert eng.cache is None
    eng.wake_up()
    assert len(eng.generate([[3, 4]], SamplingParams(max_new_tokens=2))) == 1


def test_engine_eos_and_continuous_batching(tiny):
    eng = RolloutEngine(tiny, max_num_seqs=8, max_model_len=128, sync_interval=2)
    prompts = [[10 + i, 11, 12] for i in range(10)]          # 10 requests x n=2 > 8 slots -> several admission rounds
    outs = eng.generate(prompts, SamplingParams(n=2, temperature=1.0, max_new_tokens=5, eos_token_id=7, seed=3))
    assert len(outs) == 20
    for o in outs:
        if o.finish_reason == "stop":
            assert o.token_ids[-1] == 7
        else:
            assert len(o.token_ids) == 5
    with pytest.raises(ValueError):
        eng.generate([[1] * 200], SamplingParams(max_new_tokens=5))


def test_flat_store_adamw_matches_torch(tiny):
    m1 = build_model(get_config("tiny"), dtype=torch.float32, seed=1)
    m2 = build_model(get_config("tiny"), dtype=torch.float32, seed=1)
    store = FlatParamStore(m1)
    opt = torch.optim.AdamW(m2.parameters(), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    ids = torch.randint(3, 1000, (12,), generator=torch.Generator().manual_seed(0))   # not the process-wide stream
    info = SeqInfo([12])
    for _ in range(3):
        for m in (m1, m2):
            lp, _ = m.logprobs(ids, info.positions, info, torch.roll(ids, -1))
            (-lp.mean()).backward()
        norm = store.step(lr=1e-3, max_grad_norm=1.0)
        store.zero_grad()
        ref_norm = torch.nn.utils.clip_grad_norm_(m2.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        assert norm.item() == pytest.approx(ref_norm.item(), rel=1e-4)
    for (n1, p1), (_, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        torch.testing.assert_close(p1, p2, rtol=1e-4, atol=1e-6, msg=n1)


def test_nonfinite_gradient_skips_the_step():
    m = build_model(get_config("tiny"), dtype=torch.float32, seed=2)
    store = FlatParamStore(m)
    before = store.flat_param.clone()
    store.flat_grad.fill_(float("nan"))
    store.step(lr=1.0)
    assert torch.equal(store.flat_param, before)


def test_lr_schedules():
    cfg = parse_config(["actor_rollout_ref.actor.optim.lr=1.0", "actor_rollout_ref.actor.optim.lr_warmup_steps=2",
                        "actor_rollout_ref.actor.optim.warmup_style=cosine"]).actor_rollout_ref.actor.optim
    assert lr_at_step(cfg, 0, 10) == 0.5 and lr_at_step(cfg, 1, 10) == 1.0
    assert lr_at_step(cfg, 10, 10) == pytest.approx(0.0, abs=1e-6)
    cfg.warmup_style = "constant"
    assert lr_at_step(cfg, 7, 10) == 1.0
    # the keys of the Megatron parameter scheduler
    mg = parse_config(["actor_rollout_ref.actor.optim.lr=1.0", "actor_rollout_ref.actor.optim.lr_warmup_steps=4",
                       "actor_rollout_ref.actor.optim.lr_warmup_init=0.2", "actor_rollout_ref.actor.optim.min_lr=0.1",
                       "actor_rollout_ref.actor.optim.lr_decay_style=cosine",
                       "actor_rollout_ref.actor.optim.lr_decay_steps=14"]).actor_rollout_ref.actor.optim
    assert lr_at_step(mg, 0, 100, megatron=True) == pytest.approx(0.4) and lr_at_step(mg, 3, 100, megatron=True) == 1.0
    assert lr_at_step(mg, 9, 100, megatron=True) == pytest.approx(0.1 + 0.9 * 0.5)      # half way down the cosine
    assert lr_at_step(mg, 14, 100, megatron=True) == 0.1 and lr_at_step(mg, 50, 100, megatron=True) == 0.1
    mg.lr_decay_style = "linear"
    assert lr_at_step(mg, 9, 100, megatron=True) == pytest.approx(0.55)
    mg.lr_decay_style = "constant"
    assert lr_at_step(mg, 9, 100, megatron=True) == 1.0


def test_hf_roundtrip_and_sharded_checkpoint(tmp_path, tiny):
    save_hf_model(tiny, str(tmp_path / "hf"))
    assert DecoderConfig.from_pretrained(str(tmp_path / "hf")).hidden_size == 128
    m2 = build_model(get_config("tiny"), dtype=torch.float32, seed=99)
    load_hf_weights(m2, str(tmp_path / "hf"))
    for (n, a), (_, b) in zip(tiny.named_parameters(), m2.named_parameters()):
        assert torch.equal(a, b), n
    m3 = build_model(get_config("tiny"), dtype=torch.float32, seed=5)
    s3 = FlatParamStore(m3)
    s3.flat_grad.normal_()
    s3.step(lr=1e-3)
    mgr = ShardedCheckpointManager(m3, s3, m3.cfg, contents=["model", "optimizer", "extra", "hf_model"])
    mgr.save(str(tmp_path / "ck"), global_step=4, extra={"opt_step": 1})
    assert os.path.exists(tmp_path / "ck" / "huggingface" / "model.safetensors")
    m4 = build_model(get_config("tiny"), dtype=torch.float32, seed=6)
    s4 = FlatParamStore(m4)
    extra = ShardedCheckpointManager(m4, s4, m4.cfg).load(str(tmp_path / "ck"))
    assert extra["global_step"] == 4 and extra["opt_step"] == 1
    assert torch.equal(s3.flat_param, s4.flat_param) and torch.equal(s3.exp_avg_sq, s4.exp_avg_sq)
    assert s4.step_count == 1
    # load_contents without the optimizer: weights are taken, Adam state starts fresh from them
    m5 = build_model(get_config("tiny"), dtype=torch.float32, seed=7)
    s5 = FlatParamStore(m5)
    extra = ShardedCheckpointManager(m5, s5, m5.cfg).load(str(tmp_path / "ck"), contents=["model"])
    assert torch.equal(s3.flat_param, s5.flat_param) and s5.step_count == 0 and float(s5.exp_avg_sq.abs().sum()) == 0.0
    assert torch.equal(s5.master, s5.flat_param[s5.lo:s5.hi].float()) and extra == {"global_step": 4}
    from siirl_b200.dag_worker.checkpoint_manager import CheckpointManager
    ck = parse_config(["actor_rollout_ref.actor.checkpoint.save_contents=[model,hf_model]"]).actor_rollout_ref.actor.checkpoint
    assert CheckpointManager._save_contents(ck) == ["model", "hf_model"]
    ck = parse_config(["actor_rollout_ref.actor.checkpoint.contents=[model]"]).actor_rollout_ref.actor.checkpoint
    assert CheckpointManager._save_contents(ck) == ["model"]


def test_reward_managers_place_score_at_last_valid_token():
    tok = SyntheticTokenizer()
    resp = torch.tensor([tok.encode("12") + [2, 0], tok.encode("7") + [2, 0, 0]])
    prompts = torch.tensor([tok.encode("5+7="), tok.encode("3+4=")])
    am = torch.cat([torch.ones(2, 4, dtype=torch.long), torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])], -1)
    b = Batch({"prompts": prompts, "responses": resp, "attention_mask": am},
              {"data_source": ["synthetic/arith"] * 2, "reward_model": [{"ground_truth": "12"}, {"ground_truth": "8"}]})
    r = NaiveRewardManager(tok)(b)
    assert r.tolist() == [[0, 0, 1.0, 0], [0, 0, 0, 0]]
    cfg = parse_config(["reward_model.overlong_buffer.enable=True", "reward_model.overlong_buffer.len=2"])
    d = DAPORewardManager(tok, max_resp_len=4, overlong_buffer_cfg=cfg.reward_model.overlong_buffer)(b)
    assert d[0, 2].item() == pytest.approx(1.0 - 0.5)        # length 3, expected 2 -> exceed 1 of buffer 2


def test_kv_arena_in_borrowed_memory_gives_the_same_tokens():
    """The engine may place KV blocks in a lent buffer (the trainer's idle gradient memory): same greedy output, the
    lent buffer is clobbered, and after sleep() nothing of it is referenced."""
    import torch

    from siirl_b200.engine.rollout.native_engine import RolloutEngine, SamplingParams
    from siirl_b200.models.config import get_config
    from siirl_b200.models.decoder import build_model
    cfg = get_config("tiny")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=2)
    prompts = [[5 + (3 * i + j) % 900 for j in range(10 + 7 * i)] for i in range(3)]
    sp = SamplingParams(n=2, temperature=0.0, max_new_tokens=9, ignore_eos=True)
    plain = RolloutEngine(model, max_num_seqs=8, max_model_len=128, num_blocks=24)
    want = [o.token_ids for o in plain.generate(prompts, sp)]
    eng = RolloutEngine(model, max_num_seqs=8, max_model_len=128, num_blocks=24)
    eng.sleep()
    per_layer = 24 * 2 * cfg.num_kv_heads * 64 * cfg.head_dim
    lent = torch.full((per_layer + 100,), float("nan"))          # room for ONE of the two layers, filled with NaN
    eng.borrowed = lent
    eng.wake_up()
    assert eng.kv_layout == {"blocks": 24, "layers_in_borrowed_memory": 1}
    assert eng.cache[0].data_ptr() == lent.data_ptr()
    got = [o.token_ids for o in eng.generate(prompts, sp)]
    assert got == want
    assert not torch.isnan(lent[:per_layer]).any() and float(lent[:per_layer].abs().sum()) > 0
    eng.sleep()
    assert eng.cache is None


def test_parameter_sharded_store_matches_replicated_on_gloo_ranks():
    """ZeRO-3 style store (``fsdp_config.sharding=zero3``) against the replicated one, two gloo ranks."""
    import subprocess
    import sys
    from siirl_b200.execution.scheduler.launch import find_free_port
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, Z3_DEVICE="cpu", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(find_free_port()), os.path.join(here, "zero3_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "ZERO3_OK" in out.stdout


def test_hybrid_sharded_stores_match_full_sharding_on_four_gloo_ranks():
    """``fsdp_size=2`` on four ranks: state sharded inside pairs of ranks, replicated across the pairs; the replicated-
    weights store and the parameter-sharded store both reproduce the four-way sharded run."""
    import subprocess
    import sys
    from siirl_b200.execution.scheduler.launch import find_free_port
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, Z3_DEVICE="cpu", Z3_HYBRID="2", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", str(find_free_port()), os.path.join(here, "zero3_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "ZERO3_OK" in out.stdout


def test_reward_model_reencodes_with_its_own_tokenizer_and_template():
    """A reward model with another chat template scores the re-rendered conversation and the score lands on the
    response's last valid token of the policy batch."""
    from siirl_b200.engine.workers import RewardModelWorker

    class RmTok(SyntheticTokenizer):
        def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=False, **_):
            text = "".join(f"[{m['role']}] {m['content']} ;" for m in messages)
            return self.encode(text) if tokenize else text

    cfg = parse_config(["reward_model.enable=True", "reward_model.model.arch_preset=tiny", "reward_model.max_length=64",
                        "reward_model.model.random_init=True", "trainer.device=cpu"])
    src, dst = SyntheticTokenizer(1024), RmTok(1024)
    w = RewardModelWorker(cfg.reward_model, None, torch.device("cpu"), None, 1, input_tokenizer=src, rm_tokenizer=dst)
    w.init_model()
    P = 8
    prompt = torch.tensor([[0, 0] + src.encode("1+2=?a")] * 3)
    resp = torch.tensor([src.encode("3") + [2, 0, 0, 0, 0], src.encode("12") + [2, 0, 0, 0], src.encode("123456")])
    rmask = torch.tensor([[1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0], [1] * 6])
    am = torch.cat([(prompt != 0).long(), rmask], 1)
    b = Batch({"input_ids": torch.cat([prompt, resp], 1), "attention_mask": am, "responses": resp,
               "response_mask": rmask}, None, {})
    assert w.switches_template
    rm_in = w.switch_chat_template(b)
    texts = [dst.decode(rm_in["input_ids"][i][rm_in["attention_mask"][i].bool()].tolist()) for i in range(3)]
    assert texts == ["[user] 1+2=?a ;[assistant] 3 ;", "[user] 1+2=?a ;[assistant] 12 ;",
                     "[user] 1+2=?a ;[assistant] 123456 ;"]
    scores = w.compute_rm_score(b)["rm_scores"]
    nz = scores.nonzero().tolist()
    assert nz == [[0, 1], [1, 2], [2, 5]]
    assert len({round(float(scores[i, j]), 6) for i, j in nz}) == 3       # three different conversations
    # same tokenizer on both sides: the policy's token ids are scored as they are
    w2 = RewardModelWorker(cfg.reward_model, None, torch.device("cpu"), None, 1, input_tokenizer=src)
    w2.init_model()
    assert not w2.switches_template
    assert w2.compute_rm_score(b)["rm_scores"].nonzero().tolist() == nz


def test_chunked_prefill_and_prefix_cache_give_the_same_tokens(tiny):
    """Prompts longer than the token budget enter the cache in chunks, and a second round of requests that repeat the
    first round's prompts (a multi-turn conversation re-sending its history) reuses the cached prompt blocks; greedy
    tokens equal the plain engine's in every mode."""
    cfg = get_config("tiny")
    m = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 1000, (n,), generator=g).tolist() for n in (300, 70, 200, 129)]
    ext = [p + [7, 8, 9] for p in prompts]
    sp = SamplingParams(n=2, temperature=0.0, max_new_tokens=6, ignore_eos=True)
    plain = RolloutEngine(m, max_num_seqs=8, max_model_len=512, num_blocks=64, enable_prefix_caching=False)
    want, want2 = ([o.token_ids for o in plain.generate(ps, sp)] for ps in (prompts, ext))
    chunked = RolloutEngine(m, max_num_seqs=8, max_model_len=512, num_blocks=64, max_num_batched_tokens=100,
                            enable_chunked_prefill=True, enable_prefix_caching=False)
    assert [o.token_ids for o in chunked.generate(prompts, sp)] == want
    assert chunked.stats["prefill_tokens"] == sum(len(p) for p in prompts)
    cached = RolloutEngine(m, max_num_seqs=8, max_model_len=512, num_blocks=64)
    assert [o.token_ids for o in cached.generate(prompts, sp)] == want
    assert [o.token_ids for o in cached.generate(ext, sp)] == want2
    assert cached.stats["prefix_cache_hit_tokens"] == 256 + 64 + 192 + 128       # every full prompt block was reused
    both = RolloutEngine(m, max_num_seqs=8, max_model_len=512, num_blocks=64, max_num_batched_tokens=64,
                         enable_chunked_prefill=True)
    assert [o.token_ids for o in both.generate(prompts, sp)] == want
    assert [o.token_ids for o in both.generate(ext, sp)] == want2
    # parked blocks are evicted when the free list runs dry: a small arena still serves new prompts
    small = RolloutEngine(m, max_num_seqs=4, max_model_len=512, num_blocks=14)
    for round_ in range(3):
        ps = [torch.randint(3, 1000, (150,), generator=g).tolist() for _ in range(2)]
        outs = small.generate(ps, SamplingParams(n=1, temperature=0.0, max_new_tokens=4, ignore_eos=True))
        assert len(outs) == 2 and all(len(o.token_ids) == 4 for o in outs)
    assert small.alloc.num_free == 14


def test_cache_free_engine_equals_the_paged_engine_and_serves_latent_attention():
    """``rollout.name=hf``: generation through the training forward gives the paged engine's greedy tokens and
    log-probs; it also serves the multi-head-latent-attention family, which has no paged-cache kernel."""
    from siirl_b200.engine.rollout.recompute_engine import RecomputeEngine
    model = build_model(get_config("tiny"), dtype=torch.float32, device="cpu", seed=1)
    prompts = [[5, 6, 7, 8], [9, 10, 11], [100, 200, 300, 400, 500]]
    sp = SamplingParams(n=2, temperature=0.0, max_new_tokens=7, eos_token_id=2)
    a = RecomputeEngine(model, max_num_seqs=4).generate(prompts, sp)
    eng = RolloutEngine(model, max_num_seqs=8, max_model_len=64)
    eng.wake_up()
    b = eng.generate(prompts, sp)
    assert [(o.prompt_index, o.sample_index, o.token_ids) for o in a] == \
        [(o.prompt_index, o.sample_index, o.token_ids) for o in b]
    assert max(abs(x - y) for o, p in zip(a, b) for x, y in zip(o.logprobs, p.logprobs)) < 1e-5
    mla = build_model(get_config("tiny-deepseek-v3"), dtype=torch.float32, device="cpu", seed=2)
    outs = RecomputeEngine(mla).generate(prompts[:2], SamplingParams(n=1, temperature=1.0, max_new_tokens=5, seed=3))
    assert [len(o.token_ids) for o in outs] == [5, 5] and all(o.finish_reason == "length" for o in outs)


@pytest.mark.parametrize("preset", ["tiny-deepseek-v3", "tiny-kimi-vl"])
def test_latent_cache_engine_equals_the_cache_free_engine(preset):
    """Multi-head latent attention: decoding against the cache of compressed latents (key / value expansion folded
    into query and output) gives the tokens and log-probs of recomputing the whole prefix with expanded keys and
    values; two waves, samples of a prompt sharing its prefill, EOS stops."""
    from siirl_b200.engine.rollout.latent_engine import LatentCacheEngine
    from siirl_b200.engine.rollout.recompute_engine import RecomputeEngine
    cfg = get_config(preset)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=4)
    prompts = [[5, 6, 7, 8, 9, 10], [9, 10, 11], [100, 200, 300, 400, 500], [7, 7, 7, 7]]
    for sp in (SamplingParams(n=2, temperature=0.0, max_new_tokens=9, eos_token_id=2),
               SamplingParams(n=1, temperature=0.0, max_new_tokens=4, ignore_eos=True)):
        want = RecomputeEngine(model, max_num_seqs=16).generate(prompts, sp)
        # 4 slots: two prompts x two samples per wave; 8 prompt tokens per prefill pass: one prompt at a time
        eng = LatentCacheEngine(model, max_num_seqs=4, max_model_len=32, max_num_batched_tokens=8)
        got = eng.generate(prompts, sp)
        assert eng.cache is None                                              # woke up for the call, asleep again
        assert [(o.prompt_index, o.sample_index, o.token_ids, o.finish_reason) for o in got] == \
            [(o.prompt_index, o.sample_index, o.token_ids, o.finish_reason) for o in want]
        assert max(abs(x - y) for o, p in zip(got, want) for x, y in zip(o.logprobs, p.logprobs)) < 1e-4
    if cfg.moonvit is not None:                     # image features enter through the prompt's placeholder rows
        v = cfg.moonvit
        gen = torch.Generator().manual_seed(0)
        n_img = 4 * 6 // v.merge ** 2
        mm = [{"pixel_values": torch.randn(24, 3 * v.patch_size ** 2, generator=gen),
               "image_grid_thw": torch.tensor([[1, 4, 6]])}, None]
        vp = [[5, 6] + [cfg.image_token_id] * n_img + [8, 9], [9, 10, 11]]
        sp = SamplingParams(n=2, temperature=0.0, max_new_tokens=6, ignore_eos=True)
        want = RecomputeEngine(model).generate(vp, sp, mm_inputs=mm)
        got = LatentCacheEngine(model, max_num_seqs=4, max_model_len=32).generate(vp, sp, mm_inputs=mm)
        assert [o.token_ids for o in got] == [o.token_ids for o in want]
    assert eng.stats["decode_steps"] > 0 and eng.cache_bytes() == cfg.num_layers * 4 * 32 * (cfg.kv_lora_rank + cfg.qk_rope_head_dim) * 2
