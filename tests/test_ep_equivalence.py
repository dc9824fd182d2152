"""Expert-parallel / sharded runs reproduce the gradients of the unsharded model.

Tiny Mixtral (2 layers, hidden 256, 4 heads / 2 KV heads, 4 experts of FFN 512,
top-2, vocab 1024), fp32, two gloo ranks on CPU, 2 sequences of 128 tokens per
rank with the first 40% of every sequence label-masked.  The reference for every
mode is a single process that owns all experts and averages the two ranks' losses.
"""
import pytest
import torch

from dist_utils import run_distributed
from moe_distributed_training_b200 import MixtralConfig
from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, collate_packed


def _rank_batch(cfg, rank):
    ds = SyntheticInstructionDataset(cfg.vocab_size, 2, fixed_len=128, seed=0, rank=rank)
    return collate_packed([ds[0], ds[1]])


def _collect(engine):
    """{qualified name: full gradient} for dense params; local MoE grads keyed by module path."""
    out = {}
    for u in engine.runner.all_units():
        out.update(engine.runner.full_state(u, grads=True))
    for name, p in engine.model.named_parameters():
        if ".block_sparse_moe." in name and p.grad is not None:
            out[name] = p.grad.clone()
    return {k: v.double() for k, v in out.items()}


def _run(rank, world, mode, steps):
    from moe_distributed_training_b200.train.engine import build_engine
    torch.manual_seed(0)
    cfg = MixtralConfig.tiny()
    kw = dict(dtype=torch.float32, device_type="cpu", learning_rate=1e-3, max_grad_norm=None, seed=0,
              lr_scheduler_type="constant")
    if mode == "ep":
        eng = build_engine(cfg, ep_size=world, **kw)
    elif mode == "ep-pool":
        import os
        os.environ["MDT_RESIDENT_PARAMS"] = "0"     # gather per use through the buffer pool
        eng = build_engine(cfg, ep_size=world, **kw)
        assert not eng.runner.resident
    elif mode == "ep-keep-activations":
        eng = build_engine(cfg, ep_size=world, activation_checkpointing=False, **kw)
        assert eng.runner.resident and not eng.runner.recompute
    elif mode == "ep-lora-keep-activations":
        eng = build_engine(cfg, ep_size=world, use_lora="all", activation_checkpointing=False, **kw)
        assert not eng.runner.recompute
    elif mode == "tp":
        eng = build_engine(cfg, ep_size=2, use_tp_sharding=True, **kw)
    elif mode == "tp-lora":
        eng = build_engine(cfg, ep_size=2, use_tp_sharding=True, use_lora="all", **kw)
    elif mode == "fsdp":
        eng = build_engine(cfg, ep_size=1, **kw)
    elif mode == "fsdp-lora":
        # decoder blocks (frozen experts included) are created block by block inside the sharding layer, with the
        # attention adapters added while the blocks are still on the meta device
        eng = build_engine(cfg, ep_size=1, use_lora="attn-only", **kw)
    elif mode == "ep-lora":
        eng = build_engine(cfg, ep_size=world, use_lora="all", **kw)
    else:
        raise ValueError(mode)
    if mode in ("tp", "tp-lora"):
        # tensor-parallel peers see the same batch (train_accelerate_fsdp2.py:346-382)
        dp_rank = rank // 2
        mbs = [_rank_batch(cfg, dp_rank)]
    else:
        mbs = [_rank_batch(cfg, rank)]
    losses = []
    for s in range(steps):
        loss = eng.forward_backward(mbs[0], 1.0)
        eng.runner.reduce_gradients()
        losses.append(float(loss))
        if s < steps - 1:
            eng.optimizer.step(); eng.optimizer.zero_grad(set_to_none=True)
    grads = _collect(eng)
    ep_rank = rank if mode not in ("tp", "tp-lora") else rank % 2
    return losses, grads, ep_rank


def _reference(n_batches, use_lora="none"):
    from moe_distributed_training_b200.train.engine import build_engine
    torch.manual_seed(0)
    cfg = MixtralConfig.tiny()
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", max_grad_norm=None, seed=0, use_lora=use_lora)
    losses = [float(eng.forward_backward(_rank_batch(cfg, r), 1.0 / n_batches)) for r in range(n_batches)]
    eng.runner.reduce_gradients()
    return losses, _collect(eng), cfg


def _expert_slice(ref, name, cfg, ep_rank, ep, tp=False):
    g = ref[name]
    E, F, H = cfg.num_local_experts, cfg.intermediate_size, cfg.hidden_size
    if ("lora_A" in name or "lora_B" in name) and tp:
        # tensor-parallel experts: the FFN dim of every expert is sliced; the factor on the hidden side is whole
        Fl = F // ep
        w = name.rsplit(".", 1)[-1]
        if "lora_B" in name and w in ("w1", "w3"):
            return g[:, :, ep_rank * Fl:(ep_rank + 1) * Fl]
        if "lora_A" in name and w == "w2":
            return g[:, ep_rank * Fl:(ep_rank + 1) * Fl]
        return g
    if "lora_A" in name or "lora_B" in name:
        El = E // ep
        return g[ep_rank * El:(ep_rank + 1) * El]
    if tp:
        Fl = F // ep
        return g.view(E, F, H)[:, ep_rank * Fl:(ep_rank + 1) * Fl].reshape(-1, H)
    El = E // ep
    return g.view(E, F, H)[ep_rank * El:(ep_rank + 1) * El].reshape(-1, H)


def _compare(ref_grads, grads, cfg, ep_rank, ep, tp=False, atol=2e-6):
    assert set(grads) == set(ref_grads), set(grads) ^ set(ref_grads)
    for name, g in grads.items():
        r = ref_grads[name]
        if ".experts." in name:
            r = _expert_slice(ref_grads, name, cfg, ep_rank, ep, tp)
        assert g.shape == r.shape, (name, g.shape, r.shape)
        err = (g - r).abs().max().item()
        assert err <= atol + 1e-4 * r.abs().max().item(), f"{name}: max abs err {err}"


def test_ep2_matches_unsharded():
    ref_losses, ref_grads, cfg = _reference(2)
    res = run_distributed(_run, 2, "ep", 1)
    for rank, (losses, grads, ep_rank) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank]) < 1e-5
        _compare(ref_grads, grads, cfg, ep_rank, 2)


def test_ep2_gather_per_use_matches_unsharded():
    """Parameters re-gathered for every use of a block (buffer pool) instead of resident full copies."""
    ref_losses, ref_grads, cfg = _reference(2)
    res = run_distributed(_run, 2, "ep-pool", 1)
    for rank, (losses, grads, ep_rank) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank]) < 1e-5
        _compare(ref_grads, grads, cfg, ep_rank, 2)


def test_ep2_without_recomputation_matches_unsharded():
    """Blocks run under autograd directly (activations kept) and give the same gradients."""
    ref_losses, ref_grads, cfg = _reference(2)
    res = run_distributed(_run, 2, "ep-keep-activations", 1)
    for rank, (losses, grads, ep_rank) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank]) < 1e-5
        _compare(ref_grads, grads, cfg, ep_rank, 2)
    ref_losses, ref_grads, cfg = _reference(2, use_lora="all")
    res = run_distributed(_run, 2, "ep-lora-keep-activations", 1)
    for rank, (losses, grads, ep_rank) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank]) < 1e-5
        _compare(ref_grads, grads, cfg, ep_rank, 2)


def test_single_rank_without_recomputation_matches_recomputation():
    from moe_distributed_training_b200.train.engine import build_engine
    _, ref_grads, cfg = _reference(1)
    torch.manual_seed(0)
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", max_grad_norm=None, seed=0, activation_checkpointing=False)
    assert not eng.runner.recompute
    eng.forward_backward(_rank_batch(cfg, 0), 1.0)
    eng.runner.reduce_gradients()
    grads = _collect(eng)
    assert set(grads) == set(ref_grads)
    for name, g in grads.items():
        assert (g - ref_grads[name]).abs().max().item() <= 2e-6 + 1e-4 * ref_grads[name].abs().max().item(), name


def test_fsdp2_no_ep_matches_unsharded():
    ref_losses, ref_grads, cfg = _reference(2)
    res = run_distributed(_run, 2, "fsdp", 1)
    for rank, (losses, grads, _) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank]) < 1e-5
        # experts were sharded like dense parameters: full_state returned whole tensors
        for name, g in grads.items():
            err = (g - ref_grads[name]).abs().max().item()
            assert err < 2e-6 + 1e-4 * ref_grads[name].abs().max().item(), name


def test_fsdp2_no_ep_lora_attn_matches_unsharded():
    ref_losses, ref_grads, cfg = _reference(2, use_lora="attn-only")
    res = run_distributed(_run, 2, "fsdp-lora", 1)
    for rank, (losses, grads, _) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank]) < 1e-5
        assert set(grads) == set(ref_grads) and grads
        for name, g in grads.items():
            err = (g - ref_grads[name]).abs().max().item()
            assert err < 2e-6 + 1e-4 * ref_grads[name].abs().max().item(), name


def test_ep2_lora_all_matches_unsharded():
    ref_losses, ref_grads, cfg = _reference(2, use_lora="all")
    res = run_distributed(_run, 2, "ep-lora", 1)
    for rank, (losses, grads, ep_rank) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank]) < 1e-5
        _compare(ref_grads, grads, cfg, ep_rank, 2)


def test_tp2_dp2_expert_lora_matches_unsharded():
    """Tensor-parallel experts with per-expert adapters (the reference's `ParallelMLP` LoRA wrapper, peft_utils.py:144-277):
    factors on the sliced FFN side are sliced with it, the others are whole on every rank and their gradients are summed
    over the tensor-parallel group (the reference leaves them unreduced, train_accelerate_fsdp2.py:291-298)."""
    ref_losses, ref_grads, cfg = _reference(2, use_lora="all")
    res = run_distributed(_run, 4, "tp-lora", 1)
    for rank, (losses, grads, ep_rank) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank // 2]) < 1e-5
        _compare(ref_grads, grads, cfg, ep_rank, 2, tp=True)


@pytest.mark.slow
def test_tp2_dp2_matches_unsharded():
    ref_losses, ref_grads, cfg = _reference(2)
    res = run_distributed(_run, 4, "tp", 1)
    for rank, (losses, grads, ep_rank) in enumerate(res):
        assert abs(losses[0] - ref_losses[rank // 2]) < 1e-5
        _compare(ref_grads, grads, cfg, ep_rank, 2, tp=True)


def _dtensor_views(rank, world):
    from moe_distributed_training_b200.train.engine import build_engine
    cfg = MixtralConfig.tiny()
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", ep_size=world, seed=0)
    moe = eng.model.model.layers[0].block_sparse_moe
    views = moe.as_dtensors()
    full = {k: v.full_tensor().clone() for k, v in views.items()}
    local_ok = all(torch.equal(v.to_local(), dict(moe.named_parameters())[k]) for k, v in views.items())
    placements = {k: [type(p).__name__ for p in v.placements] for k, v in views.items()}
    return full, local_ok, placements


def test_expert_parameters_as_dtensors_gather_to_the_unsharded_weights():
    from moe_distributed_training_b200.train.engine import build_engine
    cfg = MixtralConfig.tiny()
    ref = build_engine(cfg, dtype=torch.float32, device_type="cpu", seed=0).model.model.layers[0].block_sparse_moe
    for full, local_ok, placements in run_distributed(_dtensor_views, 2):
        assert local_ok
        assert placements["experts.mlp.w1"] == ["Shard"] and placements["router.layer.weight"] == ["Replicate"]
        assert torch.equal(full["router.layer.weight"].float(), ref.router.layer.weight.detach().float())
        for w in ("w1", "w2", "w3"):
            assert torch.equal(full[f"experts.mlp.{w}"].float(), getattr(ref.experts.mlp, w).detach().float()), w


def _step_with_balancing(rank, world, balance):
    from moe_distributed_training_b200.train.engine import build_engine
    cfg = MixtralConfig.tiny()
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", ep_size=world, learning_rate=1e-2, max_grad_norm=None, seed=0,
                       lr_scheduler_type="constant")
    eng.balance_microbatches = balance
    ds = SyntheticInstructionDataset(cfg.vocab_size, 4, 16, 96, seed=11, rank=rank)
    mbs = [collate_packed([ex]) for ex in ds.examples]
    eng.train_step(mbs)
    dense = {}
    for u in eng.runner.all_units():
        dense.update(eng.runner.full_state(u))
    lens = None
    if balance:
        lens = [int(mb["input_ids"].numel()) for mb in eng._balance_across_ranks(mbs)]
    return {k: v.double() for k, v in dense.items()}, lens, [int(mb["input_ids"].numel()) for mb in mbs]


def test_dealing_sequences_over_ranks_by_length_leaves_the_update_unchanged():
    """Sequences change owners so that micro-batch i has nearly the same length on every rank; the global batch is the
    same set of sequences, so one optimizer step gives the same parameters as without the exchange."""
    plain = run_distributed(_step_with_balancing, 2, False)
    dealt = run_distributed(_step_with_balancing, 2, True)
    for (pa, _, _), (pb, _, _) in zip(plain, dealt):
        assert pa.keys() == pb.keys()
        for k in pa:
            assert (pa[k] - pb[k]).abs().max().item() <= 1e-5 + 1e-4 * pa[k].abs().max().item(), k
    all_lens = sorted((n for _, _, own in dealt for n in own), reverse=True)
    l0, l1 = dealt[0][1], dealt[1][1]
    assert sorted(l0 + l1, reverse=True) == all_lens                     # nothing lost, nothing duplicated
    for i in range(4):                                                    # position i holds ranks 2i and 2i+1 of the global order
        assert sorted([l0[i], l1[i]], reverse=True) == all_lens[2 * i:2 * i + 2]
