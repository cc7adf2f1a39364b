"""The pre-training recipe end to end on CPU: mmap corpus mixture, training, checkpoint, resume incl. dataloader."""
import json
import os

import numpy as np
import torch

from ksa_b200.config import get_preset
from ksa_b200.data import KaiMMapDataset, write_corpus
from ksa_b200.training.common import StepScheduler
from ksa_b200.training.lr_schedulers import get_lr_lambda
from recipes.pretrain_ksa import get_argument_parser, train


def _corpora(tmp_path, vocab):
    rng = np.random.default_rng(0)
    for name, n in (("a", 64 * 40 + 1), ("b", 64 * 25 + 1)):
        write_corpus(str(tmp_path / "data" / name), rng.integers(0, vocab, n))
    recipe = tmp_path / "mix.txt"
    recipe.write_text(f"web\t0.7\t{tmp_path / 'data' / 'a'}\ncode\t0.3\t{tmp_path / 'data' / 'b'}\n")
    ds_cfg = tmp_path / "ds.json"
    ds_cfg.write_text(json.dumps({"name": "KaiMMapDataset", "data_prefix": str(recipe), "seq_length": 64, "seed": 7,
                                  "global_batch_size": 2, "num_workers": 1}))
    return str(ds_cfg), str(recipe)


def test_blended_dataset_is_deterministic_and_resumable(tmp_path):
    _, recipe = _corpora(tmp_path, 256)
    mk = lambda: KaiMMapDataset(recipe, 64, seed=7, global_batch_size=2)
    a, b = mk(), mk()
    ia, ib = iter(a), iter(b)
    first = [next(ia) for _ in range(5)]
    assert all(torch.equal(x["input_ids"], next(ib)["input_ids"]) for x in first)
    assert first[0]["input_ids"].shape == (1, 64) and first[0]["data_domain"][0] in ("web", "code")
    state = a.state_dict()
    nxt = [next(ia)["input_ids"] for _ in range(4)]
    c = mk()
    c.load_state_dict(state)
    ic = iter(c)
    assert all(torch.equal(x, next(ic)["input_ids"]) for x in nxt)
    # sequence-length change between stages rescales the cursors
    d = KaiMMapDataset(recipe, 32, seed=7, global_batch_size=2)
    d.load_state_dict(state)
    assert sum(d.dataset.consume_sample.values()) >= 2 * sum(state["dataset_state"][k]["c_sample"]
                                                             for k in state["dataset_state"] if k not in ("rng_state", "pending_draw")) - 2


def test_dataloader_state_of_rank_0_resumes_every_rank_on_its_own_samples(tmp_path):
    """The saved state is rank 0's; a draw that was handed out only in part must continue with each rank's own
    positions of that draw, not with rank 0's."""
    _, recipe = _corpora(tmp_path, 256)
    mk = lambda r: KaiMMapDataset(recipe, 64, seed=7, global_batch_size=8, rank=r, world_size=2)
    its = [iter(mk(0)), iter(mk(1))]
    ds0 = mk(0)
    it0 = iter(ds0)
    for _ in range(2):                      # two of rank 0's four samples of the first draw
        next(it0)
    state = ds0.state_dict()
    expect = []
    for r in (0, 1):                        # uninterrupted readers: skip two, keep the next six
        for _ in range(2):
            next(its[r])
        expect.append([next(its[r])["input_ids"] for _ in range(6)])
    assert not torch.equal(expect[0][0], expect[1][0])
    for r in (0, 1):
        d = mk(r)
        d.load_state_dict(state)
        it = iter(d)
        got = [next(it)["input_ids"] for _ in range(6)]
        assert all(torch.equal(a, b) for a, b in zip(got, expect[r])), f"rank {r}"


def test_schedulers():
    wsd = get_lr_lambda("wsd", num_warmup_steps=10, num_decay_steps=10, num_training_steps=100, base_lr=1.0, min_lr=0.1)
    assert wsd(0) == 0 and wsd(5) == 0.5 and wsd(50) == 1.0 and abs(wsd(95) - 0.55) < 1e-9 and wsd(100) == 0.1
    cos = get_lr_lambda("cosine", num_warmup_steps=0, num_training_steps=100, min_lr_rate=0.1)
    assert cos(0) == 1.0 and abs(cos(100) - 0.1) < 1e-9 and abs(cos(50) - 0.55) < 1e-9
    v2 = get_lr_lambda("cosine_v2", num_warmup_steps=0, num_decay_steps=50, num_training_steps=100, min_lr_rate=0.2)
    assert abs(v2(50) - 0.2) < 1e-9 and v2(80) == 0.2
    s = StepScheduler(2, 2, 4)
    seen = []
    for _ in range(16):
        s.step()
        seen.append((s.is_gradient_accumulation_boundary(), s.should_logging(), s.should_save_checkpoint()))
    assert s.global_step == 8 and sum(x[1] for x in seen) == 4 and sum(x[2] for x in seen) == 2


def test_recipe_trains_checkpoints_and_resumes(tmp_path):
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "summary_token_begin": 256,
                                               "head_dim": 16, "summary_chunk_size": 16})
    mc = tmp_path / "model.json"
    cfg.save(str(mc))
    ds_cfg, _ = _corpora(tmp_path, 256)
    out = tmp_path / "run"
    base = ["--model-config", str(mc), "--dataset-config", ds_cfg, "--output-dir", str(out), "--learning-rate", "3e-3",
            "--lr-scheduler-type", "constant", "--logging-per-step", "2", "--seed", "1", "--model-dtype", "float32",
            "--save-checkpoint-per-step", "4", "--enable-dataset-checkpointing"]
    r1 = train(get_argument_parser().parse_args(base + ["--num-training-steps", "8", "--disable-chunked-loss"]))
    assert r1["steps"] == 8 and (out / "latest").read_text() == "global_step8"
    assert (out / "global_step8" / "dataloader_state.pt").exists() and (out / "metrics.csv").exists()
    # the resumed leg keeps master weights and moments in host memory (--cpu-offload) and recomputes the feed-forward
    # blocks in the backward pass
    r2 = train(get_argument_parser().parse_args(base + ["--num-training-steps", "12", "--checkpoint-dir", str(out),
                                                        "--resume-weights", "--resume-optimizer", "--resume-dataloader",
                                                        "--cpu-offload", "--enable-gradient-checkpointing",
                                                        "--gradient-checkpointing-mode", "mlp"]))
    assert r2["steps"] == 12 and (out / "global_step12").is_dir()
    assert r2["loss"] < 5.6


def test_recipe_starts_from_an_hf_directory_with_skip_and_allow_lists(tmp_path):
    """``--model-dir`` + ``--skip-load-params`` / ``--allow-random-init-params``: the recipe loads a saved model, keeps
    the random initialisation of the named parameters and refuses a directory that lacks others."""
    import pytest
    from ksa_b200.models import get_model_class
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "summary_token_begin": 256,
                                               "head_dim": 16, "summary_chunk_size": 16})
    mc = tmp_path / "model.json"
    cfg.save(str(mc))
    ds_cfg, _ = _corpora(tmp_path, 256)
    src = get_model_class(cfg.model_class)(cfg)
    src.init_weights(seed=5)
    src.save_pretrained(str(tmp_path / "hf"))
    base = ["--model-config", str(mc), "--dataset-config", ds_cfg, "--learning-rate", "1e-3", "--lr-scheduler-type",
            "constant", "--seed", "1", "--model-dtype", "float32", "--num-training-steps", "2", "--model-dir",
            str(tmp_path / "hf")]
    r = train(get_argument_parser().parse_args(base + ["--output-dir", str(tmp_path / "a"), "--skip-load-params",
                                                       "_summary,summary_embedding"]))
    assert r["steps"] == 2
    # a directory without the summary parameters: refused unless they are named
    dense = {k: v for k, v in src.get_hf_state_dict().items() if "summary" not in k}
    from ksa_b200.models.base import save_sharded_safetensors
    save_sharded_safetensors(dense, str(tmp_path / "dense"))
    args = [a if a != str(tmp_path / "hf") else str(tmp_path / "dense") for a in base]
    with pytest.raises(RuntimeError, match="allow_random_init_params"):
        train(get_argument_parser().parse_args(args + ["--output-dir", str(tmp_path / "b")]))
    missing = [k for k in src.state_dict() if "summary" in k]
    r = train(get_argument_parser().parse_args(args + ["--output-dir", str(tmp_path / "c"), "--allow-random-init-params",
                                                       ",".join(missing)]))
    assert r["steps"] == 2


def _distill_rank(rank, world, port, argv, out_q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    try:
        r = train(get_argument_parser().parse_args(argv))
        out_q.put((rank, "ok", r))
    except Exception:  # noqa: BLE001
        import traceback
        out_q.put((rank, "fail", traceback.format_exc()))


def test_recipe_distillation_on_one_and_on_two_ranks(tmp_path):
    """``--enable-distill`` runs inside the engine's forward_backward (student + no-grad teacher, LM + KL + attention
    matching): the frozen base weights stay put, the summary parameters move, and two FSDP ranks (gloo) finish the same
    number of steps."""
    import socket
    import torch.multiprocessing as mp
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "summary_token_begin": 256,
                                               "head_dim": 16, "summary_chunk_size": 16})
    mc = tmp_path / "model.json"
    cfg.save(str(mc))
    ds_cfg, _ = _corpora(tmp_path, 256)
    base = ["--model-config", str(mc), "--dataset-config", ds_cfg, "--learning-rate", "3e-3", "--lr-scheduler-type",
            "constant", "--seed", "1", "--model-dtype", "float32", "--num-training-steps", "3", "--enable-distill",
            "--weight-decay", "0.5", "--logging-per-step", "1", "--save-checkpoint-per-step", "3"]
    r = train(get_argument_parser().parse_args(base + ["--output-dir", str(tmp_path / "one")]))
    assert r["steps"] == 3 and r["loss"] == r["loss"]
    from ksa_b200.models import get_model_class
    from ksa_b200.training.checkpoint import dcp_to_state_dict
    from ksa_b200.tools.convert import flatten_model_state
    tree = flatten_model_state(dcp_to_state_dict(str(tmp_path / "one" / "global_step3")))
    init = get_model_class(cfg.model_class)(cfg)
    init.init_weights(seed=1)
    muse0 = init.muse_state_dict()
    assert torch.equal(tree["model.layers.0.attn.q_proj.weight"], muse0["model.layers.0.attn.q_proj.weight"].float())
    assert not torch.equal(tree["model.layers.0.attn.q_proj_summary.weight"],
                           muse0["model.layers.0.attn.q_proj_summary.weight"].float())
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    argv = base + ["--output-dir", str(tmp_path / "two")]
    procs = [ctx.Process(target=_distill_rank, args=(rk, 2, port, argv, q)) for rk in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    for rank, status, info in res:
        assert status == "ok", f"rank {rank}: {info}"
        assert info["steps"] == 3


def test_worker_loader_resumes_at_the_next_unconsumed_sample(tmp_path):
    """A worker process prefetches ahead of the trainer; the state that comes with each batch lets a resume continue
    with the sample after the last one the trainer took."""
    from ksa_b200.data import ResumableLoader
    _, recipe = _corpora(tmp_path, 256)
    mk = lambda: KaiMMapDataset(recipe, 64, seed=7, global_batch_size=4)
    plain = iter(mk())
    expect = [next(plain)["input_ids"] for _ in range(9)]
    loader = ResumableLoader(mk(), num_workers=1, prefetch_factor=4)
    it = iter(loader)
    got = [next(it)["input_ids"] for _ in range(5)]
    assert all(torch.equal(a, b) for a, b in zip(got, expect[:5]))
    state = loader.state_dict()
    del it, loader
    resumed = ResumableLoader(mk(), num_workers=1)
    resumed.load_state_dict(state)
    it = iter(resumed)
    rest = [next(it)["input_ids"] for _ in range(4)]
    assert all(torch.equal(a, b) for a, b in zip(rest, expect[5:]))


def test_recipe_logs_per_source_loss_and_tensorboard(tmp_path):
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "summary_token_begin": 256,
                                               "head_dim": 16, "summary_chunk_size": 16})
    mc = tmp_path / "model.json"
    cfg.save(str(mc))
    ds_cfg, _ = _corpora(tmp_path, 256)
    out = tmp_path / "run"
    r = train(get_argument_parser().parse_args([
        "--model-config", str(mc), "--dataset-config", ds_cfg, "--output-dir", str(out), "--learning-rate", "1e-3",
        "--lr-scheduler-type", "constant", "--logging-per-step", "2", "--seed", "1", "--model-dtype", "float32",
        "--num-training-steps", "6", "--monitor-datasource-loss", "--num-workers", "1"]))
    assert r["steps"] == 6
    rows = (out / "metrics.csv").read_text()
    assert "domain_loss/web" in rows or "domain_loss/code" in rows
    assert "datasource_tokens/" in rows and "perf/step_elapsed" in rows
    events = [f for f in os.listdir(out / "log") if f.startswith("events.out.tfevents")]
    assert events, "no TensorBoard event file"


def test_dataset_resume_on_every_rank_for_random_mixtures_and_save_points(tmp_path):
    """Any number of sources and weights, sequence length, world size and save point: a dataset restored from rank 0's
    state continues on every rank with exactly the samples of an uninterrupted reader, also after a second save."""
    import copy
    from hypothesis import given, settings, strategies as st

    counter = [0]

    @settings(max_examples=15, deadline=None)
    @given(nsrc=st.integers(1, 4), L=st.sampled_from([16, 32]), world=st.sampled_from([1, 2, 4]),
           per_rank=st.sampled_from([1, 2, 4]), k=st.integers(0, 20), m=st.integers(1, 12), seed=st.integers(0, 1000))
    def run(nsrc, L, world, per_rank, k, m, seed):
        counter[0] += 1
        rng = np.random.default_rng(seed)
        rows = []
        for i in range(nsrc):
            prefix = str(tmp_path / f"c{counter[0]}_{i}")
            write_corpus(prefix, rng.integers(0, 500, L * int(rng.integers(3, 30)) + 1))
            rows.append(f"d{i}\t{0.05 + float(rng.random())}\t{prefix}")
        mix = tmp_path / f"mix{counter[0]}.txt"
        mix.write_text("\n".join(rows) + "\n")
        mk = lambda r: KaiMMapDataset(str(mix), L, seed=seed, global_batch_size=world * per_rank, rank=r,
                                      world_size=world)
        d0 = mk(0)
        it0 = iter(d0)
        for _ in range(k):
            next(it0)
        state = copy.deepcopy(d0.state_dict())
        for r in range(world):
            ref = iter(mk(r))
            for _ in range(k):
                next(ref)
            d = mk(r)
            d.load_state_dict(copy.deepcopy(state))
            it = iter(d)
            for j in range(m):
                assert torch.equal(next(it)["input_ids"], next(ref)["input_ids"]), (r, j)
        d = mk(0)
        d.load_state_dict(copy.deepcopy(state))
        it = iter(d)
        for _ in range(m):
            next(it)
        again = mk(0)
        again.load_state_dict(copy.deepcopy(d.state_dict()))
        ref = iter(mk(0))
        for _ in range(k + m):
            next(ref)
        it2 = iter(again)
        for j in range(4):
            assert torch.equal(next(it2)["input_ids"], next(ref)["input_ids"]), j
    run()
