"""CPU unit tests of the small components: routing plan, router, collator, CLI, schedules, flags."""
import pytest
import torch

from moe_distributed_training_b200.ops import reference


def test_plan_is_a_stable_padded_counting_sort():
    top = torch.tensor([[1, 0], [1, 2], [0, 1], [2, 1]], dtype=torch.int32)
    plan = reference.make_plan(top, 4, block=4)
    assert plan.tokens_per_expert.tolist() == [2, 4, 2, 0]
    assert plan.padded_offsets.tolist() == [0, 4, 8, 12, 12]
    # expert 1 receives slots 0, 2, 5, 7 in that (stable) order
    assert plan.dest_row[[0, 2, 5, 7]].tolist() == [4, 5, 6, 7]
    assert plan.src_slot[:12].tolist() == [1, 4, -1, -1, 0, 2, 5, 7, 3, 6, -1, -1]
    x = torch.arange(4, dtype=torch.float32)[:, None].repeat(1, 3)
    xg = reference.gather_rows(x, plan.src_slot, 2)
    assert xg[:12, 0].tolist() == [0, 2, 0, 0, 0, 1, 2, 3, 1, 3, 0, 0]
    w = torch.full((4, 2), 0.5)
    assert torch.allclose(reference.combine_rows(xg, plan.dest_row, w, 2), x)


def test_router_matches_definition():
    torch.manual_seed(0)
    x, w = torch.randn(50, 32), torch.randn(8, 32)
    s, wt, idx = reference.router(x, w, 2, True)
    ref = (x @ w.t()).softmax(-1)
    tw, ti = ref.topk(2, -1)
    assert torch.equal(idx.long(), ti)
    assert torch.allclose(wt, tw / tw.sum(-1, keepdim=True))
    assert torch.allclose(wt.sum(-1), torch.ones(50))


def test_collator_masks_prompt_and_pads():
    from moe_distributed_training_b200.data.collator import DataCollatorForCompletionOnlyLM
    c = DataCollatorForCompletionOnlyLM([7, 8], pad_token_id=0)
    b = c([{"input_ids": [1, 2, 7, 8, 5, 6]}, {"input_ids": [3, 7, 8, 4]}, {"input_ids": [1, 2, 3]}])
    assert b["input_ids"].shape == (3, 6)
    assert b["labels"][0].tolist() == [-100, -100, -100, -100, 5, 6]
    assert b["labels"][1].tolist() == [-100, -100, -100, 4, -100, -100]
    assert b["labels"][2].tolist() == [-100] * 6
    assert b["attention_mask"][1].tolist() == [1, 1, 1, 1, 0, 0]


def test_synthetic_data_shape():
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset
    ds = SyntheticInstructionDataset(1000, 20, 128, 1024, seed=1)
    for ex in ds.examples:
        n = ex["input_ids"].numel()
        assert 128 <= n <= 1024
        k = int(0.4 * n)
        assert (ex["labels"][:k] == -100).all() and (ex["labels"][k:] == ex["input_ids"][k:]).all()


def test_cli_parses_fire_style_flags():
    from moe_distributed_training_b200.cli import parse_kwargs

    def main(a: int = 1, flag: bool = False, name: str = "x", lr: float = 1e-5, deg: int = None):
        pass
    kw = parse_kwargs(main, ["--a", "3", "--flag", "True", "--name=abc", "--lr", "5e-5", "--deg", "4"])
    assert kw == {"a": 3, "flag": True, "name": "abc", "lr": 5e-5, "deg": 4}
    assert parse_kwargs(main, ["--flag"]) == {"flag": True}
    with pytest.raises(SystemExit):
        parse_kwargs(main, ["--nope", "1"])


def test_linear_schedule_decays_to_zero():
    from moe_distributed_training_b200.optim.schedulers import get_scheduler
    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=1.0)
    s = get_scheduler("linear", opt, 2, 10)
    lrs = []
    for _ in range(10):
        lrs.append(opt.param_groups[0]["lr"]); opt.step(); s.step()
    assert lrs[0] == 0.0 and lrs[2] == 1.0 and abs(lrs[6] - 0.5) < 1e-9 and opt.param_groups[0]["lr"] == 0.0


def test_flag_validation_follows_the_reference_rules():
    from moe_distributed_training_b200.train.run import validate_flags
    with pytest.raises(ValueError):
        validate_flags(False, True, False, "none", 8, None)      # scattermoe needs a sharding mode
    with pytest.raises(ValueError):
        validate_flags(True, False, True, "none", 8, None)       # exactly one of megablocks / tp
    assert validate_flags(True, False, False, "all", 8, None) == 8   # expert_degree defaults to world size
    assert validate_flags(True, True, False, "attn-only", 8, 4) == 4
    assert validate_flags(False, False, False, "none", 8, None) == 1


def test_get_moe_kwargs_and_constants():
    from megablocks_utils.shard_moe_utils import (DIM_EXPERT, KEY_DATA_PARALLEL, KEY_EXPERT_PARALLEL, KEY_EXPERTS,
                                                  KEY_ROUTER, get_moe_kwargs)
    from moe_distributed_training_b200 import MixtralConfig
    kw = get_moe_kwargs(MixtralConfig.mixtral_8x7b(), bf16=True, mlp_impl="scattermoe")
    assert kw["ffn_hidden_size"] == 14336 and kw["moe_num_experts"] == 8 and kw["moe_top_k"] == 2
    assert kw["moe_expert_model_parallelism"] and kw["moe_normalize_expert_weights"] is True
    assert (KEY_DATA_PARALLEL, KEY_EXPERT_PARALLEL, DIM_EXPERT) == ("data_parallel", "expert_parallel", 0)
    assert (KEY_ROUTER, KEY_EXPERTS) == ("router.layer.weight", "experts.mlp")


def test_moe_block_contract_and_param_names():
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.models.mixtral import MixtralForCausalLM
    cfg = MixtralConfig.tiny()
    m = MixtralForCausalLM(cfg)
    names = dict(m.named_parameters())
    assert names["model.layers.0.block_sparse_moe.router.layer.weight"].shape == (4, 256)
    assert names["model.layers.1.block_sparse_moe.experts.mlp.w2"].shape == (4 * 512, 256)
    out, aux = m.model.layers[0].block_sparse_moe(torch.randn(2, 5, 256))
    assert out.shape == (2, 5, 256) and aux is None


def test_parallel_linear_lora_matches_expert_model():
    """The scenario of the reference's unit test: 10 tokens, 2 experts, fixed routing, LoRA r=16/alpha=32."""
    from scattermoe_utils.parallel_linear_lora import parallel_linear_lora
    torch.manual_seed(42)
    E, K, N, r, alpha = 2, 128, 16, 16, 32
    X = torch.randn(10, K, requires_grad=True)
    W = torch.randn(E, K, N) * 0.1
    A = (torch.randn(E, K, r) * 0.1).requires_grad_(True)
    B = (torch.randn(E, r, N) * 0.1).requires_grad_(True)
    sorted_expert_idxs = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1, 1, 1])
    sorted_scattered_idxs = torch.tensor([4, 6, 8, 9, 0, 1, 2, 3, 5, 7])
    out = parallel_linear_lora(X, W, A, B, r, alpha, 1, sorted_expert_idxs, sorted_scattered_idxs)
    Xr, Ar, Br = (t.detach().clone().requires_grad_(True) for t in (X, A, B))
    ref = torch.zeros(10, N)
    for e in range(E):
        rows = sorted_scattered_idxs[sorted_expert_idxs == e]
        ref[rows] = Xr[rows] @ W[e] + (alpha / r) * (Xr[rows] @ Ar[e]) @ Br[e]
    assert torch.allclose(out, ref, atol=1e-5)
    go = torch.randn(10, N)
    out.backward(go); ref.backward(go)
    for a, b in ((X, Xr), (A, Ar), (B, Br)):
        assert torch.allclose(a.grad, b.grad, atol=1e-5)
    # top-2 fan-out with gates, and the primitives under the reference's names
    from scattermoe_utils.kernels.ops import group_bwd_AB, padded_block_indices, scatter2scatter_lora
    pbi, eo = padded_block_indices(torch.tensor([0] * 300 + [1] * 200), 2)
    assert pbi.tolist() == [0, 128, 256, 300, 428] and eo.tolist() == [300, 500]
    y = scatter2scatter_lora(X.detach(), W, A.detach(), B.detach(), alpha / r, sorted_expert_idxs, sorted_scattered_idxs, 1)
    assert torch.allclose(y, ref.detach(), atol=1e-5)
    xs = X.detach()[sorted_scattered_idxs]
    dA, dB = group_bwd_AB(go[sorted_scattered_idxs], xs, A.detach(), B.detach(), alpha / r, torch.tensor([4, 10]), 2)
    assert torch.allclose(dA, Ar.grad, atol=1e-5) and torch.allclose(dB, Br.grad, atol=1e-5)


def test_launcher_translates_an_accelerate_config(tmp_path):
    """accelerate.yaml + accelerator_config.json -> torchrun command line and environment."""
    import json, os, subprocess, sys
    import pytest
    from moe_distributed_training_b200 import launch
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = launch._load_yaml(os.path.join(root, "accelerate.yaml"))
    accel = json.load(open(os.path.join(root, "accelerator_config.json")))
    plan = launch.plan_launch(cfg, ["train_fsdp1.py", "--use_megablocks_sharding"], num_processes=4, accelerator_config=accel)
    assert "--nproc-per-node=4" in plan.command and "--nnodes=1" in plan.command
    assert plan.command[-2:] == ["train_fsdp1.py", "--use_megablocks_sharding"]
    assert plan.command[plan.command.index("--master-addr") + 1] == "127.0.0.1"
    assert plan.env == {"MDT_RESIDENT_PARAMS": "0", "MDT_SYNC_EACH_BATCH": "1"}
    cfg2 = dict(cfg, fsdp_config=dict(cfg["fsdp_config"], fsdp_sharding_strategy="SHARD_GRAD_OP"))
    assert launch.plan_launch(cfg2, ["x.py"]).env["MDT_RESIDENT_PARAMS"] == "1"
    for bad in ({"fsdp_sharding_strategy": 3}, {"fsdp_offload_params": True}):
        with pytest.raises(ValueError):
            launch.plan_launch(dict(cfg, fsdp_config=dict(cfg["fsdp_config"], **bad)), ["x.py"])
    out = subprocess.run([sys.executable, "-m", "moe_distributed_training_b200.launch", "--config_file",
                          os.path.join(root, "accelerate.yaml"), "--num_processes", "2", "--dry_run", "train_fsdp1.py"],
                         capture_output=True, text=True, cwd=root, check=True)
    assert "--nproc-per-node=2" in json.loads(out.stdout)["command"]


def test_text_dataset_masks_the_prompt_with_a_local_tokenizer(tmp_path):
    """data.json records -> token ids with everything up to the response template label-masked."""
    import json
    pytest = __import__("pytest")
    tokenizers = pytest.importorskip("tokenizers")
    transformers = pytest.importorskip("transformers")
    from moe_distributed_training_b200.train.run import _load_text_dataset
    words = ["<unk>", "<s>", "</s>", "###", "Response", "Instruction", ":", "hello", "world", "answer", "is", "42", "what", "Question", "Answer"]
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<s>", eos_token="</s>")
    fast.save_pretrained(str(tmp_path))
    data = tmp_path / "data.json"
    data.write_text(json.dumps([{"output": "### Instruction : what is hello world ### Response : answer is 42"}]))
    out = _load_text_dataset(str(data), str(tmp_path), 64)
    assert len(out) == 1
    ids, labels = out[0]["input_ids"].tolist(), out[0]["labels"].tolist()
    assert ids == [3, 5, 6, 12, 10, 7, 8, 3, 4, 6, 9, 10, 11]
    assert labels[:9] == [-100] * 9 and labels[9:] == ids[9:]       # prompt and template masked, answer kept
    assert _load_text_dataset(str(tmp_path / "missing.json"), str(tmp_path), 64) is None
    # alpaca-style records are formatted "### Question: ... ### Answer: ..." and masked up to the answer
    alp = tmp_path / "alpaca.json"
    alp.write_text(json.dumps([{"instruction": "what is hello", "input": "", "output": "answer is 42"}]))
    out = _load_text_dataset(str(alp), str(tmp_path), 64)
    labels = out[0]["labels"].tolist()
    assert labels[-3:] == [9, 10, 11] and all(v == -100 for v in labels[:-3])


def test_gemm_tiling_choice_without_a_gpu():
    """The host-side rule that picks between the 128-row, CTA-pair and tall GEMM tilings (pure arithmetic)."""
    build = pytest.importorskip("moe_distributed_training_b200.ops.build")
    try:
        ext = build.load()
    except Exception:  # noqa: BLE001
        pytest.skip("extension not built")

    def choose(mode, M, N, K, K_l=0, G=1, cap=0, dual=False, c_fp32=False, acc=False, offs=False, policy=3, hint=0, sms=148):
        return ext.gemm_choose_tiling(mode, M, N, K, K_l, G, cap, dual, c_fp32, acc, offs, policy, hint, sms)
    TILE128, PAIR, TALL = 0, 1, 2
    assert choose(0, 8192, 8192, 8192) == TALL                       # many waves, long depth
    assert choose(0, 576, 4096, 4096) == TILE128                     # attention projection of one micro-batch: one wave
    assert choose(0, 576, 1024, 4096) == TILE128
    assert choose(0, 576, 16, 4096) == TILE128                       # narrow outputs never use 256-wide tiles
    assert choose(0, 1152, 32000, 4096) == TILE128                   # lm_head: 4.5 tall tiles per column block, no gain
    # expert GEMMs inside the exchange: buffers sized for 16 384 rows, ~1 300 expected
    # 11 x 16 = 176 tiles on 148 SMs: the 128-row kernel shares the 28 tiles of its second round among all SMs along the
    # depth; without that sharing two rounds would be needed and the tall tiling wins
    assert choose(1, 0, 4096, 14336, cap=16384, offs=True, hint=1300) == TILE128
    old = ext.gemm_set_split(0)
    try:
        assert choose(1, 0, 4096, 14336, cap=16384, offs=True, hint=1300) == TALL
    finally:
        ext.gemm_set_split(old)
    assert choose(1, 0, 4096, 14336, cap=16384, offs=True, hint=500) == TILE128   # one wave either way
    assert choose(2, 14336, 4096, 0, cap=16384, acc=True, offs=True, hint=1152) == TILE128   # weight gradient: short depth
    assert choose(0, 8192, 8192, 8192, policy=0) == TILE128
    assert choose(0, 8192, 8192, 8192, policy=2) == PAIR
    assert choose(0, 300, 520, 200, policy=4) == TALL
    assert choose(0, 300, 128, 200, policy=4) == TILE128             # 128-wide outputs: only the 128-row kernel exists


def test_profile_trace_flag_writes_a_trace(tmp_path):
    from moe_distributed_training_b200.train.run import run_training
    out = tmp_path / "traces"
    run_training(model_preset="tiny", model_name_or_path=None, device_type="cpu", load_model_dtype="float32",
                 gradient_accumulation_steps=2, max_steps=3, num_synthetic_examples=8, data_path=str(tmp_path / "none.json"),
                 profile_trace=str(out), profile_steps=1)
    files = list(out.glob("trace_rank*.json"))
    assert len(files) == 1 and files[0].stat().st_size > 1000


def test_fsdp1_entry_accepts_the_reference_readme_command(tmp_path):
    """Every flag of the reference README's FSDP1 command line (README.md:58-80) is understood."""
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "train_fsdp1.py"), "--accelerator_config", os.path.join(root, "accelerator_config.json"),
           "--data_path", str(tmp_path / "data.json"), "--torch_dtype", "float32", "--bf16", "False", "--output_dir", str(tmp_path / "results"),
           "--num_train_epochs", "1", "--per_device_train_batch_size", "1", "--per_device_eval_batch_size", "1",
           "--gradient_accumulation_steps", "2", "--gradient_checkpointing", "True", "--evaluation_strategy", "no",
           "--save_strategy", "no", "--learning_rate", "5e-5", "--lr_scheduler_type", "linear", "--logging_steps", "1",
           "--use_megablocks_sharding", "True", "--model_preset", "tiny", "--device_type", "cpu", "--num_synthetic_examples", "4"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "train_runtime" in p.stdout


def test_aux_loss_from_router_statistics_matches_the_definition():
    """With a load-balancing weight the router keeps its per-expert histogram / score sums; the layer's aux loss built
    from them equals E * sum_e f_e P_e stated directly, and it back-propagates into the router."""
    from moe_distributed_training_b200.models.mixtral import moe_args_from_config
    from moe_distributed_training_b200.moe.layer import dMoE
    from moe_distributed_training_b200.ops.reference import load_balancing_loss
    from moe_distributed_training_b200 import MixtralConfig
    cfg = MixtralConfig.tiny()
    cfg.router_aux_loss_coef = 0.01
    moe = dMoE(moe_args_from_config(cfg, torch.float32, "cpu"))
    x = torch.randn(2, 24, cfg.hidden_size)
    out, _ = moe(x)
    aux = moe.aux_loss()
    scores, top = moe.last_scores
    want = 0.01 * load_balancing_loss(scores, top, cfg.num_local_experts, cfg.num_experts_per_tok)
    assert torch.allclose(aux, want, rtol=1e-6)
    assert moe.router.last_stats is not None and int(moe.router.last_stats[:cfg.num_local_experts].sum()) == top.numel()
    aux.backward()
    assert moe.router.layer.weight.grad is not None and float(moe.router.layer.weight.grad.abs().sum()) > 0
