"""HF Mixtral safetensors ingest / export and resumable training state (CPU)."""
import json
import os

import torch

from dist_utils import run_distributed
from moe_distributed_training_b200 import MixtralConfig
from moe_distributed_training_b200.checkpoint import hf_safetensors as hfst


def _write_tiny_hf_checkpoint(path, cfg, seed=0):
    """A sharded HF-layout checkpoint (two files + index) with random weights."""
    g = torch.Generator().manual_seed(seed)
    H, F, E, V = cfg.hidden_size, cfg.intermediate_size, cfg.num_local_experts, cfg.vocab_size
    qd, kvd = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    t = {}
    r = lambda *s: torch.randn(*s, generator=g) * 0.02
    t["model.embed_tokens.weight"] = r(V, H)
    t["model.norm.weight"] = torch.ones(H)
    t["lm_head.weight"] = r(V, H)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        t[f"{p}.input_layernorm.weight"] = torch.ones(H)
        t[f"{p}.post_attention_layernorm.weight"] = torch.ones(H)
        t[f"{p}.self_attn.q_proj.weight"] = r(qd, H)
        t[f"{p}.self_attn.k_proj.weight"] = r(kvd, H)
        t[f"{p}.self_attn.v_proj.weight"] = r(kvd, H)
        t[f"{p}.self_attn.o_proj.weight"] = r(H, qd)
        t[f"{p}.block_sparse_moe.gate.weight"] = r(E, H)
        for e in range(E):
            t[f"{p}.block_sparse_moe.experts.{e}.w1.weight"] = r(F, H)
            t[f"{p}.block_sparse_moe.experts.{e}.w2.weight"] = r(H, F)
            t[f"{p}.block_sparse_moe.experts.{e}.w3.weight"] = r(F, H)
    keys = sorted(t)
    half = len(keys) // 2
    files = {"model-00001-of-00002.safetensors": {k: t[k] for k in keys[:half]},
             "model-00002-of-00002.safetensors": {k: t[k] for k in keys[half:]}}
    hfst.save_sharded(files, path)
    cfg.save_pretrained(path)
    return t


def test_key_mapper_orders_experts_and_rejects_unknown_keys():
    wm = {"model.layers.0.block_sparse_moe.gate.weight": "a",
          "model.layers.0.block_sparse_moe.experts.1.w1.weight": "b",
          "model.layers.0.block_sparse_moe.experts.0.w1.weight": "a",
          "model.layers.0.block_sparse_moe.experts.0.w2.weight": "a",
          "model.layers.0.block_sparse_moe.experts.1.w2.weight": "a",
          "model.layers.0.block_sparse_moe.experts.0.w3.weight": "a",
          "model.layers.0.block_sparse_moe.experts.1.w3.weight": "b",
          "model.layers.1.block_sparse_moe.gate.weight": "a"}
    out = hfst.get_router_experts_sharded_safetensor(wm, "model.layers.0", "block_sparse_moe")
    assert out["router.layer.weight"] == [("model.layers.0.block_sparse_moe.gate.weight", "a")]
    assert [k for k, _ in out["experts.mlp.w1"]] == [f"model.layers.0.block_sparse_moe.experts.{e}.w1.weight" for e in (0, 1)]
    assert out["experts.mlp.w3"][1][1] == "b"
    wm["model.layers.0.block_sparse_moe.experts.0.w9.weight"] = "a"
    try:
        hfst.get_router_experts_sharded_safetensor(wm, "model.layers.0", "block_sparse_moe")
        raise AssertionError("unknown key accepted")
    except ValueError:
        pass


def test_single_process_load_and_export_roundtrip(tmp_path):
    from moe_distributed_training_b200.checkpoint.state import save_model
    from moe_distributed_training_b200.train.engine import build_engine
    cfg = MixtralConfig.tiny()
    src = str(tmp_path / "src")
    tensors = _write_tiny_hf_checkpoint(src, cfg)
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", checkpoint=src)
    moe = eng.model.model.layers[1].block_sparse_moe
    F, H = cfg.intermediate_size, cfg.hidden_size
    w2 = moe.experts.mlp.w2.view(cfg.num_local_experts, F, H)
    assert torch.equal(w2[3], tensors["model.layers.1.block_sparse_moe.experts.3.w2.weight"].t())
    assert torch.equal(moe.router.layer.weight, tensors["model.layers.1.block_sparse_moe.gate.weight"])
    out = str(tmp_path / "out")
    save_model(eng, out)
    wm = hfst.read_weight_map(out)
    assert set(wm) == set(tensors)
    from safetensors import safe_open
    for k, fname in wm.items():
        with safe_open(os.path.join(out, fname), framework="pt") as f:
            assert torch.equal(f.get_tensor(k), tensors[k]), k


def test_assign_mlp_v2_weights_fills_a_module_from_the_key_map(tmp_path):
    """The reference's loader entry point: key map of one layer -> router and expert weights of a MoE module."""
    from megablocks_utils.shard_moe_utils import assign_mlp_v2_weights, get_router_experts_sharded_safetensor
    from moe_distributed_training_b200.models.mixtral import moe_args_from_config
    from moe_distributed_training_b200.moe.layer import dMoE
    cfg = MixtralConfig.tiny()
    src = str(tmp_path / "src")
    tensors = _write_tiny_hf_checkpoint(src, cfg)
    settings = get_router_experts_sharded_safetensor(hfst.read_weight_map(src), "model.layers.0", "block_sparse_moe")
    moe = dMoE(moe_args_from_config(cfg, torch.float32, "cpu"))
    assign_mlp_v2_weights(moe, src, settings, None, None)
    F, H, E = cfg.intermediate_size, cfg.hidden_size, cfg.num_local_experts
    assert torch.equal(moe.router.layer.weight, tensors["model.layers.0.block_sparse_moe.gate.weight"])
    for e in range(E):
        assert torch.equal(moe.experts.mlp.w1.view(E, F, H)[e], tensors[f"model.layers.0.block_sparse_moe.experts.{e}.w1.weight"])
        assert torch.equal(moe.experts.mlp.w2.view(E, F, H)[e], tensors[f"model.layers.0.block_sparse_moe.experts.{e}.w2.weight"].t())
        assert torch.equal(moe.experts.mlp.w3.view(E, F, H)[e], tensors[f"model.layers.0.block_sparse_moe.experts.{e}.w3.weight"])


def _ep_roundtrip(rank, world, src, out):
    from moe_distributed_training_b200.checkpoint.state import save_model
    from moe_distributed_training_b200.train.engine import build_engine
    cfg = MixtralConfig.from_pretrained(src)
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", ep_size=world, checkpoint=src)
    mlp = eng.model.model.layers[0].block_sparse_moe.experts.mlp
    assert mlp.w1.shape == (cfg.num_local_experts // world * cfg.intermediate_size, cfg.hidden_size)
    save_model(eng, out)
    return True


def test_ep2_load_shards_and_export_roundtrip(tmp_path):
    cfg = MixtralConfig.tiny()
    src, out = str(tmp_path / "src"), str(tmp_path / "out")
    tensors = _write_tiny_hf_checkpoint(src, cfg)
    run_distributed(_ep_roundtrip, 2, src, out)
    wm = hfst.read_weight_map(out)
    assert set(wm) == set(tensors)
    from safetensors import safe_open
    for k, fname in wm.items():
        with safe_open(os.path.join(out, fname), framework="pt") as f:
            assert torch.equal(f.get_tensor(k), tensors[k]), k


def test_training_state_resume(tmp_path):
    from moe_distributed_training_b200.checkpoint.state import load_training_state, save_training_state
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, batches
    from moe_distributed_training_b200.train.engine import build_engine
    cfg = MixtralConfig.tiny()
    ds = SyntheticInstructionDataset(cfg.vocab_size, 6, 16, 32)
    mbs = list(batches(ds, 1))
    a = build_engine(cfg, dtype=torch.float32, device_type="cpu", learning_rate=1e-3, num_training_steps=3)
    a.train_step(mbs[:2]); a.train_step(mbs[2:4])
    save_training_state(a, str(tmp_path), 2)
    la = float(a.train_step(mbs[4:6])["loss"])
    b = build_engine(cfg, dtype=torch.float32, device_type="cpu", learning_rate=1e-3, num_training_steps=3)
    assert load_training_state(b, str(tmp_path)) == 2
    lb = float(b.train_step(mbs[4:6])["loss"])
    assert abs(la - lb) < 1e-6
    for p, q in zip(a.model.parameters(), b.model.parameters()):
        assert torch.allclose(p, q, atol=1e-7)


def test_adapter_save_uses_peft_names(tmp_path):
    from moe_distributed_training_b200.checkpoint.state import save_adapter
    from moe_distributed_training_b200.train.engine import build_engine
    from safetensors.torch import load_file
    cfg = MixtralConfig.tiny()
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", use_lora="all")
    save_adapter(eng, str(tmp_path))
    t = load_file(str(tmp_path / "adapter_model.safetensors"))
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" in t
    assert t["base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight"].shape == (16, cfg.hidden_size)
    k = "base_model.model.model.layers.1.block_sparse_moe.experts.2.w2.lora_B.weight"
    assert t[k].shape == (cfg.hidden_size, 16)
    assert json.load(open(tmp_path / "adapter_config.json"))["r"] == 16


def _train_save_load_adapter(rank, world, out_dir):
    """Train adapters for a step, save them, load them into a freshly built engine, compare every adapter value."""
    from moe_distributed_training_b200.checkpoint.state import load_adapter, save_adapter
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, batches
    from moe_distributed_training_b200.train.engine import build_engine
    cfg = MixtralConfig.tiny()
    kw = dict(dtype=torch.float32, device_type="cpu", use_lora="all", learning_rate=1e-2, ep_size=world if world > 1 else None)
    a = build_engine(cfg, seed=0, **kw)
    ds = SyntheticInstructionDataset(cfg.vocab_size, 2, 16, 32, rank=rank)
    a.train_step(list(batches(ds, 1)))            # lora_B leaves zero: the saved values are not the initial ones
    save_adapter(a, out_dir)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    b = build_engine(cfg, seed=1, **kw)           # other initial adapters
    pa = {n: p for n, p in a.model.named_parameters() if p.requires_grad}
    pb = {n: p for n, p in b.model.named_parameters() if p.requires_grad}
    assert pa.keys() == pb.keys() and pa
    assert any(not torch.equal(pa[n], pb[n]) for n in pa)
    load_adapter(b, out_dir)
    for n in pa:
        assert torch.equal(pa[n].detach(), pb[n].detach()), n
    # a tensor in the file that matches nothing is an error, not a silent skip
    return sorted(os.listdir(out_dir))


def test_adapter_roundtrip_single_rank(tmp_path):
    files = _train_save_load_adapter(0, 1, str(tmp_path))
    assert "adapter_model.safetensors" in files and not [f for f in files if "rank" in f]


def test_adapter_roundtrip_two_ranks_expert_parallel(tmp_path):
    files = run_distributed(_train_save_load_adapter, 2, str(tmp_path))[0]
    assert "adapter_model.safetensors" in files and not [f for f in files if "rank" in f]
    from safetensors.torch import load_file
    t = load_file(str(tmp_path / "adapter_model.safetensors"))
    cfg = MixtralConfig.tiny()
    for e in range(cfg.num_local_experts):          # experts of both ranks are in the one file
        assert f"base_model.model.model.layers.0.block_sparse_moe.experts.{e}.w1.lora_A.weight" in t


def test_load_adapter_rejects_a_file_that_does_not_fit(tmp_path):
    from moe_distributed_training_b200.checkpoint.state import load_adapter, save_adapter
    from moe_distributed_training_b200.train.engine import build_engine
    from safetensors.torch import load_file, save_file
    cfg = MixtralConfig.tiny()
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", use_lora="attn-only")
    save_adapter(eng, str(tmp_path))
    path = str(tmp_path / "adapter_model.safetensors")
    t = load_file(path)
    dropped = sorted(t)[0]
    extra = dict(t)
    del extra[dropped]
    extra["base_model.model.model.layers.0.self_attn.nothing.lora_A.weight"] = torch.zeros(2, 2)
    save_file(extra, path)
    try:
        load_adapter(eng, str(tmp_path))
        raise AssertionError("a file with a missing and an unknown tensor was accepted")
    except KeyError as exc:
        assert "missing" in str(exc) and "unmatched" in str(exc)
