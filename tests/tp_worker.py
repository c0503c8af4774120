"""Body of the tensor-parallel checks, one process per rank (torchrun env).  ``TP_DEVICE=cpu`` runs on gloo ranks
(host logic and the all_reduce fallback), ``TP_DEVICE=cuda`` on NCCL ranks with the fused GEMM + all-reduce kernel."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from siirl_b200.engine.rollout.native_engine import RolloutEngine, SamplingParams  # noqa: E402
from siirl_b200.models.config import get_config  # noqa: E402
from siirl_b200.models.decoder import build_model  # noqa: E402
from siirl_b200.models.tp_decoder import TPDecoder  # noqa: E402
from siirl_b200.parallel.tensor_parallel import TPContext  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = os.environ.get("TP_DEVICE", "cpu") == "cuda"
    if cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl")
        dev = torch.device("cuda", torch.cuda.current_device())
        from siirl_b200.ops import lib
        from siirl_b200.parallel.symm import SymmComm
        comm = SymmComm.create(dist.group.WORLD)
    else:
        dist.init_process_group("gloo")
        dev, comm = torch.device("cpu"), None
    dtype = torch.bfloat16 if cuda else torch.float32
    H = 512
    ctx = TPContext(dist.group.WORLD, comm, max_rows=1024, max_cols=H, max_tiles=64)

    # 1. row-parallel linear == full linear, decode-sized and prefill-sized, repeated (launch epochs advance)
    g = torch.Generator().manual_seed(7)
    K = 1024 * world
    for M in (8, 64, 128, 300, 512, 1000, 8):
        x = torch.randn(M, K, generator=g).to(dev, dtype)
        w = (0.05 * torch.randn(H, K, generator=g)).to(dev, dtype)
        b = torch.randn(H, generator=g).to(dev, dtype)
        ks = K // world
        y = ctx.row_parallel_linear(x[:, rank * ks:(rank + 1) * ks].contiguous(), w[:, rank * ks:(rank + 1) * ks], b)
        want = x.float() @ w.float().t() + b.float()
        err = (y.float() - want).abs().max().item()
        tol = 0.25 if cuda else 1e-3
        assert err < tol, f"row-parallel linear M={M}: max err {err}"
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()

    # 2. tensor-parallel engine generates the same greedy tokens as the single-rank engine
    cfg = get_config("tiny-gpu" if cuda else "tiny")
    model = build_model(cfg, dtype=dtype, device=dev, seed=5)
    prompts = [[(7 * i + 3 * j) % (cfg.vocab_size - 10) + 3 for j in range(20 + 5 * i)] for i in range(4)]
    sp = SamplingParams(n=1, temperature=0.0, max_new_tokens=12, ignore_eos=True)
    ref_engine = RolloutEngine(model, max_num_seqs=8, max_model_len=128, num_blocks=32)
    want_tokens = [o.token_ids for o in ref_engine.generate(prompts, sp)]
    ref_engine.sleep()
    ctx2 = TPContext(dist.group.WORLD, comm, max_rows=1024, max_cols=cfg.hidden_size, max_tiles=64)
    tp_model = TPDecoder(model, ctx2)
    engine = RolloutEngine(tp_model, max_num_seqs=8, max_model_len=128, num_blocks=32)
    assert engine.cache[0].shape[2] == cfg.num_kv_heads // world
    outs = engine.generate(prompts, sp)
    got_tokens = [o.token_ids for o in outs]
    same = sum(int(a == b) for x, y in zip(want_tokens, got_tokens) for a, b in zip(x, y))
    total = sum(len(x) for x in want_tokens)
    # bf16 summation order differs between the sharded and the full contraction: allow a few argmax flips
    assert same >= (total if not cuda else int(0.8 * total)), (same, total, want_tokens, got_tokens)
    # weights follow the replica after an update
    with torch.no_grad():
        model.layers[0].qkv_proj_weight.mul_(0.5)
    tp_model.sync_weights()
    hq = cfg.num_heads // world * cfg.head_dim
    assert torch.equal(tp_model.layers[0].qkv_w[:hq], model.layers[0].qkv_proj_weight[rank * hq:(rank + 1) * hq])
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()
    # 2b. low-rank adapters are folded into the engine's slices: same greedy tokens as the single-rank engine, which
    #     applies base weight and adapter separately
    cfg_l = get_config("tiny-gpu" if cuda else "tiny", {"lora_rank": 8, "lora_alpha": 16.0})
    model_l = build_model(cfg_l, dtype=dtype, device=dev, seed=6)
    with torch.no_grad():
        for n_, p_ in model_l.named_parameters():
            if "_lora_B" in n_:
                p_.copy_((0.05 * torch.randn(p_.shape, generator=g)).to(dev, dtype))
    ref_l = RolloutEngine(model_l, max_num_seqs=8, max_model_len=128, num_blocks=32)
    want_l = [o.token_ids for o in ref_l.generate(prompts, sp)]
    ref_l.sleep()
    model_l.set_lora_enabled(False)
    base_l = [o.token_ids for o in RolloutEngine(model_l, max_num_seqs=8, max_model_len=128, num_blocks=32).generate(prompts, sp)]
    model_l.set_lora_enabled(True)
    assert base_l != want_l, "the adapters must change the greedy tokens for this check to mean anything"
    tp_l = TPDecoder(model_l, ctx2)
    got_l = [o.token_ids for o in RolloutEngine(tp_l, max_num_seqs=8, max_model_len=128, num_blocks=32).generate(prompts, sp)]
    same_l = sum(int(a == b) for x, y in zip(want_l, got_l) for a, b in zip(x, y))
    assert same_l >= (total if not cuda else int(0.8 * total)), (same_l, total)
    # 3. all-gather -> GEMM: weight rows sharded over the ranks, gathered inside the GEMM launch
    from siirl_b200.parallel.ag_gemm import AgLinear
    N2, K2 = 1536 * world, 640
    w_full = (0.05 * torch.randn(N2, K2, generator=g)).to(dev, dtype)
    b2 = torch.randn(N2, generator=g).to(dev, dtype)
    ag = AgLinear(dist.group.WORLD, comm, N2, K2, copiers=8, device=dev, dtype=dtype)
    ag.load_shard(w_full[rank * ag.rows:(rank + 1) * ag.rows])
    for M in (300, 64, 1000):
        x = torch.randn(M, K2, generator=g).to(dev, dtype)
        y = ag(x, b2)
        want = x.float() @ w_full.float().t() + b2.float()
        err = (y.float() - want).abs().max().item()
        assert err < (0.3 if cuda else 1e-3), f"ag_gemm M={M}: max err {err}"
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()
    # 4. Ulysses layout switches: sequence shard <-> head shard, forward values and the backward (the other pull)
    from siirl_b200.parallel.ulysses import UlyssesSP
    hq, hkv, D, Tl = 4 * world, 2 * world, 16, 24
    W = (hq + 2 * hkv) * D
    parts = [(0, hq * D), (hq * D, hkv * D), ((hq + hkv) * D, hkv * D)]
    usp = UlyssesSP(dist.group.WORLD, comm, max_elems=world * Tl * W)
    full = torch.randn(world * Tl, W, generator=g).to(dev, dtype)          # same on every rank
    mine = full[rank * Tl:(rank + 1) * Tl].clone().requires_grad_()
    heads = usp.seq_to_heads(mine, parts)
    hl, kl = hq // world * D, hkv // world * D
    want = torch.cat([full[:, rank * hl:(rank + 1) * hl], full[:, hq * D + rank * kl: hq * D + (rank + 1) * kl],
                      full[:, (hq + hkv) * D + rank * kl:(hq + hkv) * D + (rank + 1) * kl]], dim=1)
    assert torch.equal(heads.detach(), want), "seq_to_heads"
    back = usp.heads_to_seq(heads, parts)
    assert torch.equal(back.detach(), mine.detach()), "round trip"
    coef = torch.randn(Tl, W, generator=g).to(dev, dtype)
    (back * coef).sum().backward()
    assert torch.allclose(mine.grad.float(), coef.float()), "backward of the two switches is the identity map"
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()
    # 5. a decoder under sequence parallelism: local rows of the hidden states and summed parameter gradients
    #    equal the single-rank computation
    from siirl_b200.ops.attention import SeqInfo
    cfg5 = get_config("tiny-gpu" if cuda else "tiny")
    m_full = build_model(cfg5, dtype=dtype, device=dev, seed=9)
    m_sp = build_model(cfg5, dtype=dtype, device=dev, seed=9)
    width = (cfg5.num_heads + 2 * cfg5.num_kv_heads) * cfg5.head_dim
    m_sp.attach_sequence_parallel(UlyssesSP(dist.group.WORLD, comm, max_elems=512 * width))
    lens = [37, 64, 22]                                   # 123 tokens: not a multiple of the group size
    info = SeqInfo(lens, device=dev)
    ids = torch.randint(3, cfg5.vocab_size, (sum(lens),), generator=g).to(dev)
    coef = torch.randn(sum(lens), cfg5.hidden_size, generator=g).to(dev, dtype)
    h_full = m_full.forward_hidden(ids, info.positions, info)
    (h_full.float() * coef.float()).sum().backward()
    h_loc = m_sp.forward_hidden(ids, info.positions, info)
    lo, hi, pad = m_sp.sp_slice(sum(lens))
    n_real = min(hi, sum(lens)) - lo
    tol5 = 0.1 if cuda else 1e-4
    assert (h_loc[:n_real].float() - h_full[lo:lo + n_real].float()).abs().max().item() < tol5, "SP hidden rows"
    (h_loc[:n_real].float() * coef[lo:lo + n_real].float()).sum().backward()
    for (n1, p1), (_, p2) in zip(m_full.named_parameters(), m_sp.named_parameters()):
        if p1.grad is None and getattr(p1, "main_grad", None) is None:
            continue                                      # not on the path of forward_hidden (LM head)
        g2 = (p2.grad if p2.grad is not None else p2.main_grad).float().clone()
        dist.all_reduce(g2)
        g1 = (p1.grad if p1.grad is not None else p1.main_grad).float()
        err = (g1 - g2).abs().max().item()
        assert err < (0.05 * max(1.0, g1.abs().max().item()) if cuda else 1e-3), f"SP grad {n1}: {err}"
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()
    # 5b. multi-head latent attention (DeepSeek-V3 / Kimi-VL language model) under the same switch: the three
    #     operands have different head widths (query / key 48, value 32 in the tiny configuration)
    if not cuda:
        cfg5b = get_config("tiny-deepseek-v3")
        mla_full = build_model(cfg5b, dtype=dtype, device=dev, seed=11)
        mla_sp = build_model(cfg5b, dtype=dtype, device=dev, seed=11)
        wide = cfg5b.num_heads * (2 * (cfg5b.qk_nope_head_dim + cfg5b.qk_rope_head_dim) + cfg5b.v_head_dim)
        mla_sp.attach_sequence_parallel(UlyssesSP(dist.group.WORLD, comm, max_elems=512 * wide))
        hb_full = mla_full.forward_hidden(ids, info.positions, info)
        hb_loc = mla_sp.forward_hidden(ids, info.positions, info)
        assert (hb_loc[:n_real].float() - hb_full[lo:lo + n_real].float()).abs().max().item() < 1e-4, "MLA SP rows"
        (hb_full.float() * coef.float()).sum().backward()
        (hb_loc[:n_real].float() * coef[lo:lo + n_real].float()).sum().backward()
        pf, ps = dict(mla_full.named_parameters()), dict(mla_sp.named_parameters())
        for n5 in ("layers.0.kv_b_proj_weight", "layers.1.q_b_proj_weight", "layers.2.kv_a_proj_weight"):
            g2 = (ps[n5].grad if ps[n5].grad is not None else ps[n5].main_grad).float().clone()
            dist.all_reduce(g2)
            g1 = (pf[n5].grad if pf[n5].grad is not None else pf[n5].main_grad).float()
            assert (g1 - g2).abs().max().item() < 1e-3, f"MLA SP grad {n5}"
    # 6. ring (context-parallel) attention equals causal attention over the whole sequences, values and gradients
    from siirl_b200.ops.attention import attention_packed
    from siirl_b200.parallel.ring_attention import RingContext, ring_attention, split_for_context_parallel
    hq6, hkv6, d6 = 4, 2, 64
    W6 = (hq6 + 2 * hkv6) * d6
    lens6 = [128 * world, 192 * world]
    T6 = sum(lens6)
    full6 = (0.5 * torch.randn(T6, W6, generator=g)).to(dev, dtype)
    go6 = torch.randn(T6, hq6 * d6, generator=g).to(dev, dtype)
    ref_in = full6.clone().requires_grad_()
    ref_out = attention_packed(ref_in, SeqInfo(lens6, device=dev), hq6, hkv6, d6, causal=True)
    ref_out.backward(go6)
    t6 = 0.06 if cuda else 1e-4
    # on CPU ranks: once through the gathered statement, once through the block algorithms of the GPU path over an
    # emulated symmetric memory
    for zz, emu in ((False, False), (True, False)) + (() if cuda else ((False, True), (True, True))):
        rows, _, info6 = split_for_context_parallel(lens6, world, rank, device=dev, zigzag=zz)
        rc = RingContext(dist.group.WORLD, comm, max_rows=rows.numel(), qkv_width=W6, kv_width=2 * hkv6 * d6,
                         zigzag=zz, emulate=emu)
        loc = full6[rows].clone().requires_grad_()
        out6 = ring_attention(loc, rc, info6, hq6, hkv6, d6)
        out6.backward(go6[rows])
        assert (out6.float() - ref_out[rows].float()).abs().max().item() < t6, f"ring attention output (zigzag={zz}, emulated={emu})"
        assert (loc.grad.float() - ref_in.grad[rows].float()).abs().max().item() < 4 * t6, f"ring attention gradient (zigzag={zz}, emulated={emu})"
        if cuda:
            torch.cuda.synchronize()
            lib.check_status()
    # 7. a decoder under context parallelism (ring attention inside every layer): the rows this rank computes equal
    #    the single-rank hidden states, and summed parameter gradients match
    m_cp = build_model(cfg5, dtype=dtype, device=dev, seed=9)
    m_ref = build_model(cfg5, dtype=dtype, device=dev, seed=9)
    m_cp.attach_context_parallel(RingContext(dist.group.WORLD, comm, max_rows=256, qkv_width=width,
                                             kv_width=2 * cfg5.num_kv_heads * cfg5.head_dim, zigzag=True))
    lens7 = [37, 64, 23]
    info7 = SeqInfo(lens7, device=dev)
    ids7 = torch.randint(3, cfg5.vocab_size, (sum(lens7),), generator=g).to(dev)
    coef7 = torch.randn(sum(lens7), cfg5.hidden_size, generator=g).to(dev, dtype)
    ok_cp = (not cuda) or cfg5.head_dim in (64, 128)
    if ok_cp:
        h_ref = m_ref.forward_hidden(ids7, info7.positions, info7)
        (h_ref.float() * coef7.float()).sum().backward()
        h_cp = m_cp.forward_hidden(ids7, info7.positions, info7)
        loc = m_cp.local_row_index(info7, sum(lens7))
        keep = loc >= 0
        assert (h_cp[keep].float() - h_ref[loc[keep]].float()).abs().max().item() < tol5, "CP hidden rows"
        (h_cp[keep].float() * coef7[loc[keep]].float()).sum().backward()
        for (n1, p1), (_, p2) in zip(m_ref.named_parameters(), m_cp.named_parameters()):
            if p1.grad is None:
                continue
            g2 = p2.grad.float().clone()
            dist.all_reduce(g2)
            err = (p1.grad.float() - g2).abs().max().item()
            assert err < (0.05 * max(1.0, p1.grad.float().abs().max().item()) if cuda else 1e-3), f"CP grad {n1}: {err}"
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()
    # 7b. a vision-language decoder under sequence and under context parallelism: image features are written over the
    #     whole stream before the rows are divided; local rows and summed gradients (tower included) equal one rank's
    if not cuda:
        from siirl_b200.models.vision import mrope_positions
        cfgv = get_config("tiny-vl")
        grid = torch.tensor([[1, 8, 12]])
        n_img = 8 * 12 // cfgv.vision.spatial_merge_size ** 2
        seq_a = torch.cat([torch.randint(3, 900, (5,), generator=g), torch.full((n_img,), cfgv.image_token_id),
                           torch.randint(3, 900, (11,), generator=g)])
        seq_b = torch.randint(3, 900, (21,), generator=g)
        idsv = torch.cat([seq_a, seq_b]).to(dev)
        lensv = [seq_a.numel(), seq_b.numel()]
        infov = SeqInfo(lensv, device=dev)
        posv = torch.cat([mrope_positions(seq_a, cfgv.image_token_id, grid, cfgv.vision.spatial_merge_size),
                          torch.arange(seq_b.numel()).expand(3, -1)], 1).to(dev)
        coefv = torch.randn(sum(lensv), cfgv.hidden_size, generator=g).to(dev, dtype)
        for mode in ("ulysses", "ring"):
            mv_ref = build_model(cfgv, dtype=dtype, device=dev, seed=11)
            mv = build_model(cfgv, dtype=dtype, device=dev, seed=11)
            pix = torch.randn(8 * 12, mv.vision.patch_dim, generator=g).to(dev, dtype)
            wv = (cfgv.num_heads + 2 * cfgv.num_kv_heads) * cfgv.head_dim
            if mode == "ulysses":
                mv.attach_sequence_parallel(UlyssesSP(dist.group.WORLD, comm, max_elems=512 * wv))
            else:
                mv.attach_context_parallel(RingContext(dist.group.WORLD, comm, max_rows=256, qkv_width=wv,
                                                       kv_width=2 * cfgv.num_kv_heads * cfgv.head_dim, zigzag=True))
            hv_ref = mv_ref.forward_hidden(idsv, posv, infov, pixel_values=pix, image_grid_thw=grid)
            (hv_ref.float() * coefv.float()).sum().backward()
            hv = mv.forward_hidden(idsv, posv, infov, pixel_values=pix, image_grid_thw=grid)
            loc = mv.local_row_index(infov, sum(lensv))
            keep = loc >= 0
            assert (hv[keep].float() - hv_ref[loc[keep]].float()).abs().max().item() < 1e-4, f"VL hidden rows ({mode})"
            (hv[keep].float() * coefv[loc[keep]].float()).sum().backward()
            seen_tower = False
            for (n1, p1), (_, p2) in zip(mv_ref.named_parameters(), mv.named_parameters()):
                g1 = p1.grad if p1.grad is not None else getattr(p1, "main_grad", None)
                if g1 is None:
                    continue
                g2 = (p2.grad if p2.grad is not None else p2.main_grad).float().clone()
                dist.all_reduce(g2)
                assert (g1.float() - g2).abs().max().item() < 1e-3, f"VL grad {n1} ({mode})"
                seen_tower = seen_tower or n1.startswith("vision.")
            assert seen_tower
    # 8. pipeline parallelism: stages exchange activations / gradients point to point; every stage's parameter
    #    gradients equal the single-rank ones, and weight sync after an update restores identical replicas
    from siirl_b200.parallel.pipeline import PipelineContext, sync_stage_weights
    cfg8 = get_config("tiny-gpu" if cuda else "tiny", {"tie_word_embeddings": False})
    m_pp = build_model(cfg8, dtype=dtype, device=dev, seed=4)
    m_one = build_model(cfg8, dtype=dtype, device=dev, seed=4)
    pc = PipelineContext(dist.group.WORLD, cfg8.num_layers)
    m_pp.attach_pipeline_parallel(pc)
    info8 = SeqInfo([33, 50], device=dev)
    ids8 = torch.randint(3, cfg8.vocab_size, (83,), generator=g).to(dev)
    coef8 = torch.randn(83, cfg8.hidden_size, generator=g).to(dev, dtype)
    h_one = m_one.forward_hidden(ids8, info8.positions, info8)
    (h_one.float() * coef8.float()).sum().backward()
    hidden, handle = m_pp.forward_hidden_pp(ids8, info8.positions, info8)
    if pc.is_last:
        assert (hidden.float() - h_one.float()).abs().max().item() < tol5, "PP hidden"
        (hidden.float() * coef8.float()).sum().backward()
    else:
        handle.backward()
    for (n1, p1), (_, p2) in zip(m_one.named_parameters(), m_pp.named_parameters()):
        if p1.grad is None:
            continue
        if pc.owns_param(n1):
            err = (p1.grad.float() - p2.grad.float()).abs().max().item()
            assert err < (0.05 * max(1.0, p1.grad.float().abs().max().item()) if cuda else 1e-3), f"PP grad {n1}: {err}"
        else:
            assert p2.grad is None, f"{n1} is trained by another stage"
    with torch.no_grad():
        for n1, p2 in m_pp.named_parameters():
            if pc.owns_param(n1):
                p2.add_(1.0)
    sync_stage_weights(m_pp, pc)
    chk = torch.stack([p.float().sum() for p in m_pp.parameters()]).sum().reshape(1)
    parts = [torch.zeros_like(chk) for _ in range(world)]
    dist.all_gather(parts, chk)
    assert all(torch.allclose(parts[0], q) for q in parts), "replicas differ after stage weight sync"
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()
    dist.barrier()
    if rank == 0:
        print("TP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
