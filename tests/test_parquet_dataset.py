"""The parquet data path users run: row-group slices per data-parallel rank, chat-format prompts, ground truth under
``reward_model``, over-long prompts, and a GRPO step on a GSM8K-shaped file scored by the gsm8k rule."""
import json
import os
import subprocess
import sys

import pytest
import torch

pa = pytest.importorskip("pyarrow")
import pyarrow.parquet as pq  # noqa: E402

from siirl_b200.data_coordinator.dataloader import DataLoaderNode, load_tokenizer  # noqa: E402
from siirl_b200.data_coordinator.dataloader.partitioned_dataset import PartitionedRLHFDataset  # noqa: E402
from siirl_b200.params import parse_config  # noqa: E402


def _write(path, n, start=0, long_every=0, row_group_size=7):
    rows = []
    for i in range(start, start + n):
        q = f"What is {i} plus {i + 1}?" + (" please explain in great detail" * 20 if long_every and i % long_every == 0 else "")
        rows.append({"data_source": "openai/gsm8k", "prompt": [{"role": "user", "content": q}], "ability": "math",
                     "reward_model": {"style": "rule", "ground_truth": str(2 * i + 1)},
                     "extra_info": {"index": i, "split": "train"}})
    pq.write_table(pa.Table.from_pylist(rows), str(path), row_group_size=row_group_size)
    return rows


def test_row_group_slices_cover_the_files_once(tmp_path):
    _write(tmp_path / "a.parquet", 23)
    _write(tmp_path / "b.parquet", 18, start=23)
    args = [f"data.train_files=[{tmp_path / 'a.parquet'},{tmp_path / 'b.parquet'}]", f"data.val_files={tmp_path / 'b.parquet'}",
            "data.max_prompt_length=64", "actor_rollout_ref.model.arch_preset=tiny", "trainer.n_gpus_per_node=1"]
    cfg = parse_config(args)
    tok = load_tokenizer(None, 1024)
    seen = []
    for rank in range(3):
        ds = PartitionedRLHFDataset(cfg, tok, None, rank, 3, is_eval=False)
        assert len(ds) == 41 // 3                                       # training drops the remainder
        seen += [r["extra_info"]["index"] for r in ds.rows]
        item = ds[0]
        assert item["input_ids"].shape == (64,) and int(item["attention_mask"].sum()) == len(item["raw_prompt_ids"])
        assert item["data_source"] == "openai/gsm8k" and item["reward_model"]["ground_truth"] == str(2 * ds.rows[0]["extra_info"]["index"] + 1)
    assert seen == list(range(39))                                      # contiguous slices across the file boundary
    val = [PartitionedRLHFDataset(cfg, tok, None, r, 4, is_eval=True, drop_last=False) for r in range(4)]
    assert [len(v) for v in val] == [5, 5, 5, 5]                        # 18 rows: the last rank is padded
    assert sum(r["padded_duplicate"] for v in val for r in v.rows) == 2
    real = [r["extra_info"]["index"] for v in val for r in v.rows if not r["padded_duplicate"]]
    assert real == list(range(23, 41))


def test_overlong_prompts_are_filtered_or_truncated(tmp_path):
    _write(tmp_path / "a.parquet", 12, long_every=4)
    base = [f"data.train_files={tmp_path / 'a.parquet'}", "data.max_prompt_length=48",
            "actor_rollout_ref.model.arch_preset=tiny", "trainer.n_gpus_per_node=1"]
    tok = load_tokenizer(None, 1024)
    kept = PartitionedRLHFDataset(parse_config(base + ["data.filter_overlong_prompts=True"]), tok, None, 0, 1)
    assert len(kept) == 9 and all(r["extra_info"]["index"] % 4 for r in kept.rows)
    ds = PartitionedRLHFDataset(parse_config(base + ["data.truncation=left"]), tok, None, 0, 1)
    assert len(ds) == 12 and int(ds[0]["attention_mask"].sum()) == 48
    with pytest.raises(Exception):
        PartitionedRLHFDataset(parse_config(base + ["data.truncation=error"]), tok, None, 0, 1)[0]


def test_grpo_step_on_a_gsm8k_shaped_parquet_file(tmp_path):
    _write(tmp_path / "train.parquet", 32)
    _write(tmp_path / "test.parquet", 8, start=100)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(tmp_path / "log"))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    args = ["algorithm.adv_estimator=grpo", f"data.train_files={tmp_path / 'train.parquet'}",
            f"data.val_files={tmp_path / 'test.parquet'}", "data.max_prompt_length=64", "data.max_response_length=16",
            "data.train_batch_size=4", "actor_rollout_ref.model.arch_preset=tiny", "actor_rollout_ref.rollout.n=4",
            "actor_rollout_ref.rollout.max_num_seqs=16", "actor_rollout_ref.actor.ppo_mini_batch_size=4",
            "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8", "trainer.n_gpus_per_node=1", "trainer.device=cpu",
            "trainer.val_before_train=True", "trainer.test_freq=1", "trainer.logger=['jsonl']",
            "trainer.total_training_steps=2", "trainer.save_freq=-1"]
    out = subprocess.run([sys.executable, "-m", "siirl_b200.main_dag", *args], env=env, cwd=root, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    with open(tmp_path / "log" / "metrics.jsonl") as f:
        m = [json.loads(line) for line in f]
    assert any("val-core/openai/gsm8k/reward/mean@1" in r or "val-core/all/reward/mean" in r for r in m)
    steps = [r for r in m if "actor/pg_loss" in r]
    assert [r["step"] for r in steps] == [1, 2]
    assert all(r["critic/score/mean"] == 0.0 for r in steps)       # a random model never writes "#### <answer>"


def _make_hf_tokenizer(path):
    """A small word-level tokenizer saved in the Hugging Face layout (tokenizer.json + tokenizer_config.json with a
    chat template), built offline."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    words = ["<pad>", "<eos>", "<unk>", "<|user|>", "<|assistant|>", "what", "is", "plus", "?", "####"] + \
        [str(i) for i in range(200)]
    tk = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tk.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tk, pad_token="<pad>", eos_token="<eos>", unk_token="<unk>")
    fast.chat_template = ("{% for m in messages %}{{ '<|' + m['role'] + '|> ' + m['content'] + ' ' }}{% endfor %}"
                          "{% if add_generation_prompt %}{{ '<|assistant|> ' }}{% endif %}")
    fast.save_pretrained(str(path))
    return len(words)


def test_hugging_face_tokenizer_directory(tmp_path):
    """``data.tokenizer`` / ``model.path`` with tokenizer files: chat template applied, loader options honoured, new
    special tokens must fit the model's vocabulary."""
    import types
    vocab = _make_hf_tokenizer(tmp_path / "tok")
    tok = load_tokenizer(str(tmp_path / "tok"), vocab_size=vocab)
    assert tok.pad_token_id == 0 and tok.eos_token_id == 1
    rows = [{"data_source": "openai/gsm8k", "prompt": [{"role": "user", "content": f"what is {i} plus {i + 1} ?"}],
             "reward_model": {"ground_truth": str(2 * i + 1)}} for i in range(6)]
    pq.write_table(pa.Table.from_pylist(rows), str(tmp_path / "t.parquet"))
    cfg = parse_config([f"data.train_files={tmp_path / 't.parquet'}", "data.max_prompt_length=16",
                        "actor_rollout_ref.model.arch_preset=tiny", "trainer.n_gpus_per_node=1"])
    ds = PartitionedRLHFDataset(cfg, tok, None, 0, 1)
    ids = ds[2]["raw_prompt_ids"]
    assert tok.decode(ids) == "<|user|> what is 2 plus 3 ? <|assistant|>"
    assert ds[2]["input_ids"][-len(ids):].tolist() == ids and int(ds[2]["input_ids"][0]) == tok.pad_token_id   # left pad
    args = types.SimpleNamespace(use_fast_tokenizer=True, split_special_tokens=False, trust_remote_code=False,
                                 new_special_tokens="<tool>,<obs>", resize_vocab=False)
    with pytest.raises(ValueError, match="beyond the model's vocabulary"):
        load_tokenizer(str(tmp_path / "tok"), vocab_size=vocab, model_args=args)
    roomy = load_tokenizer(str(tmp_path / "tok"), vocab_size=vocab + 8, model_args=args)
    assert roomy.convert_tokens_to_ids("<tool>") == vocab and len(roomy) == vocab + 2
    # a directory without tokenizer files falls back to the synthetic tokenizer
    assert type(load_tokenizer(str(tmp_path), vocab_size=64)).__name__ == "SyntheticTokenizer"


def test_training_from_a_checkpoint_directory(tmp_path):
    """The launch line of a real run: ``model.path`` names a directory with ``config.json``, safetensors weights and
    tokenizer files; data comes from parquet files.  The policy starts from the stored weights (the reference model
    too, so the KL term starts at zero) and the exported checkpoint keeps the Hugging Face layout."""
    from siirl_b200.models.config import get_config
    from siirl_b200.models.decoder import build_model
    from siirl_b200.models.hf_io import save_hf_model
    vocab = _make_hf_tokenizer(tmp_path / "model")
    cfg = get_config("tiny", {"vocab_size": 256, "eos_token_id": 1, "pad_token_id": 0})
    assert vocab <= cfg.vocab_size
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=11)
    save_hf_model(model, str(tmp_path / "model"))
    rows = [{"data_source": "openai/gsm8k", "prompt": [{"role": "user", "content": f"what is {i} plus {i + 1} ?"}],
             "reward_model": {"ground_truth": str(2 * i + 1)}} for i in range(16)]
    pq.write_table(pa.Table.from_pylist(rows), str(tmp_path / "train.parquet"))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(tmp_path / "log"))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    args = ["algorithm.adv_estimator=grpo", f"data.train_files={tmp_path / 'train.parquet'}",
            f"data.val_files={tmp_path / 'train.parquet'}", "data.max_prompt_length=32", "data.max_response_length=12",
            "data.train_batch_size=4", f"actor_rollout_ref.model.path={tmp_path / 'model'}",
            "actor_rollout_ref.rollout.n=4", "actor_rollout_ref.rollout.max_num_seqs=16",
            "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
            "actor_rollout_ref.actor.use_kl_loss=True", "actor_rollout_ref.actor.optim.lr=1e-4",
            "actor_rollout_ref.actor.checkpoint.contents=[model,optimizer,extra,hf_model]",
            "trainer.n_gpus_per_node=1", "trainer.device=cpu", "trainer.val_before_train=False",
            "trainer.logger=['jsonl']", "trainer.total_training_steps=2", "trainer.save_freq=2",
            f"trainer.default_local_dir={tmp_path / 'ckpt'}"]
    out = subprocess.run([sys.executable, "-m", "siirl_b200.main_dag", *args], env=env, cwd=root, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    with open(tmp_path / "log" / "metrics.jsonl") as f:
        m = [json.loads(line) for line in f]
    assert [r["step"] for r in m] == [1, 2]
    assert m[0]["actor/kl_loss"] == 0.0                    # policy and reference both loaded the stored weights
    hf = tmp_path / "ckpt" / "global_step_2" / "actor_agent_0" / "huggingface"
    assert (hf / "model.safetensors").exists() and (hf / "config.json").exists() and (hf / "tokenizer.json").exists()
    from safetensors.torch import load_file
    new = load_file(str(hf / "model.safetensors"))
    old = load_file(str(tmp_path / "model" / "model.safetensors"))
    assert set(new) == set(old)
    moved = max((new[k].float() - old[k].float()).abs().max().item() for k in old)
    assert 0.0 < moved < 0.1                               # trained from the stored weights, not from a fresh init
