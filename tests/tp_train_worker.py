"""Body of the tensor-parallel TRAINING checks on gloo ranks: a decoder cut into column- / row-parallel slices (with
and without Megatron sequence parallelism, activation checkpointing and a vocabulary-parallel LM head) gives the same
log-probs, entropies and -- after gathering the slices -- the same gradients as the whole model."""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from siirl_b200.models.config import get_config
from siirl_b200.models.decoder import build_model
from siirl_b200.ops.attention import SeqInfo
from siirl_b200.parallel.megatron_tp import TPTrainContext, shard_decoder, per_tensor_generator, allreduce_sequence_parallel_grads, vocab_parallel_logprob_entropy
from siirl_b200.ops.lm_head import lm_head_logprob_entropy
def main():
    dist.init_process_group("gloo"); rank, world = dist.get_rank(), dist.get_world_size()
    cfg = get_config("tiny")
    g = torch.Generator().manual_seed(5)
    lens=[9,14,8]; ids=torch.randint(3,cfg.vocab_size,(31,),generator=g); labels=torch.randint(3,cfg.vocab_size,(31,),generator=g)
    info=SeqInfo(lens)
    for sp, vp, ckpt in ((False, False, False), (True, False, True), (False, True, False), (True, True, False)):
        full = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
        shard = build_model(cfg, dtype=torch.float32, device="cpu", seed=3, gradient_checkpointing=ckpt)
        tp = TPTrainContext(dist.group.WORLD, sequence_parallel=sp)
        shard_decoder(shard, tp, vocab_parallel=vp)
        lp, ent = full.logprobs(ids, info.positions, info, labels, temperature=0.8)
        (-(lp.mean()) + 0.01*ent.mean()).backward()
        lp2, ent2 = shard.logprobs(ids, info.positions, info, labels, temperature=0.8)
        (-(lp2.mean()) + 0.01*ent2.mean()).backward()
        allreduce_sequence_parallel_grads(shard, tp)
        assert (lp-lp2).abs().max()<1e-5 and (ent-ent2).abs().max()<1e-5, (sp,vp,(lp-lp2).abs().max())
        # gradients: gather shard grads like weights and compare
        fullg = {n:p.grad for n,p in full.named_parameters()}
        # temporarily put grads into .data to reuse the generator
        saved = {n:p.data for n,p in shard.named_parameters()}
        for n,p in shard.named_parameters(): p.data = p.grad
        for n,t in per_tensor_generator(shard, tp):
            assert t.shape == fullg[n].shape, (n, t.shape, fullg[n].shape)
            err=(t-fullg[n]).abs().max().item()
            assert err < 1e-5, (sp, vp, n, err)
        for n,p in shard.named_parameters(): p.data = saved[n]
        for n,t in per_tensor_generator(shard, tp):
            assert torch.equal(t, dict(full.named_parameters())[n].data), n
    if rank==0: print("TP_TRAIN_OK")
    dist.barrier(); dist.destroy_process_group()
main()
