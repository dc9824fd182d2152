"""Worker of the multi-GPU tests (one process per GPU, started by torch.distributed.run).

Runs the same training steps with the library token exchange ("nccl") and with the peer-memory
exchange ("fused") and writes the per-step losses and a parameter checksum of both to a JSON file.
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path, mode = sys.argv[1], sys.argv[2]
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, collate_packed
    from moe_distributed_training_b200.train.engine import build_engine
    import torch.distributed as dist
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    cfg = MixtralConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=128, num_local_experts=4, num_experts_per_tok=2)
    if mode == "rank-exit":
        return rank_exit(out_path, cfg, rank, world)
    use_lora = "all" if mode == "lora" else "none"
    ds = SyntheticInstructionDataset(cfg.vocab_size, 6, 100, 400, seed=3, rank=rank)
    mbs = [collate_packed([ex]) for ex in ds.examples]
    result = {}
    if mode.endswith("-pool"):
        # gather per use through the buffer pool (no resident copies), with matrices of the tiny model counted as
        # GEMM-only weights: the peer-memory arm then runs the all-gather with progress flags and the GEMMs that
        # wait for their weight operand chunk by chunk
        os.environ["MDT_RESIDENT_PARAMS"] = "0"
        os.environ["MDT_GEMM_ONLY_MIN_NUMEL"] = str(1 << 16)
        mode = mode[:-len("-pool")]
    for impl in ("nccl", "fused"):
        if mode == "tp":
            # tensor-parallel experts on a (dp, tp) mesh: the partial sums of the down projection are added up by the
            # library all-reduce or by the peer-memory all-reduce kernel; tensor-parallel peers share a batch
            os.environ["MDT_PEER_COLLECTIVES"] = "0" if impl == "nccl" else "1"
            eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", ep_size=2, use_tp_sharding=True, learning_rate=1e-3,
                               seed=0, lr_scheduler_type="constant")
            ds_tp = SyntheticInstructionDataset(cfg.vocab_size, 6, 100, 400, seed=3, rank=rank // 2)
            mbs = [collate_packed([ex]) for ex in ds_tp.examples]
        elif mode.startswith("fsdp"):
            # no expert parallelism: everything, experts included, is sharded; compare NCCL collectives with the
            # peer-memory all-gather / reduce-scatter kernels
            os.environ["MDT_PEER_COLLECTIVES"] = "0" if impl == "nccl" else "1"
            eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", ep_size=1, use_lora="attn-only" if mode == "fsdp-lora" else "none",
                               learning_rate=1e-3, seed=0, lr_scheduler_type="constant")
        else:
            os.environ["MDT_PEER_COLLECTIVES"] = "0" if impl == "nccl" else "1"
            eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", ep_size=world, use_lora=use_lora, learning_rate=1e-3,
                               seed=0, dispatch_impl=impl, ep_max_tokens=512, lr_scheduler_type="constant")
        losses = [float(eng.train_step(mbs[2 * s:2 * s + 2])["loss"]) for s in range(3)]
        from moe_distributed_training_b200.ops import cuda_ops
        cuda_ops.check_status(eng.device)
        chk = sum(float(p.detach().float().abs().sum()) for p in eng.model.parameters() if p.requires_grad)
        result[impl] = {"losses": losses, "checksum": chk}
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.barrier()
    dist.destroy_process_group()


def rank_exit(out_path, cfg, rank, world):
    """The last rank leaves between two steps, with none of its kernels or collectives in flight; the others learn of
    it on the host (a key in a c10d store) before they launch anything that would wait for it."""
    import time
    import torch.distributed as dist
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, collate_packed
    from moe_distributed_training_b200.train.engine import build_engine
    from moe_distributed_training_b200.utils.failure import Heartbeat, RankFailure, guarded_step
    eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", ep_size=world, learning_rate=1e-3, seed=0,
                       dispatch_impl="fused", ep_max_tokens=512, lr_scheduler_type="constant")
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 7, world, rank == 0, wait_for_workers=False)
    hb = Heartbeat(store, rank, world, limit_s=30.0)
    ds = SyntheticInstructionDataset(cfg.vocab_size, 4, 100, 300, seed=5, rank=rank)
    mbs = [collate_packed([ex]) for ex in ds.examples]
    guarded_step(eng, mbs[:2], hb)                 # a normal step: every rank stamps the store afterwards
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    outcome = {"rank": rank, "loss_ok": True}
    if rank == world - 1:
        hb.mark_failed("left between steps")
        outcome["left"] = True
    else:
        deadline = time.time() + 20.0
        while not hb.stale_ranks() and time.time() < deadline:
            time.sleep(0.05)
        try:
            guarded_step(eng, mbs[2:4], hb)        # must stop on the host, before any kernel is launched
            outcome["detected"] = []
        except RankFailure as exc:
            outcome["detected"] = exc.ranks
        from moe_distributed_training_b200.ops import cuda_ops
        torch.cuda.synchronize()
        cuda_ops.check_status(eng.device)           # no device-side wait ran out: nothing was launched
        outcome["step_count"] = eng.step_count
    with open(f"{out_path}.rank{rank}", "w") as f:
        json.dump(outcome, f)
    sys.stdout.flush()
    os._exit(0)                                     # no collective teardown: a peer is gone by design


if __name__ == "__main__":
    main()
