"""Context parallelism on CPU ranks (gloo): sharded attention and the sharded model equal the whole sequence."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ksa_b200.config import get_preset
from ksa_b200.models import get_model_class


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg(chunk, window, n_sum):
    return get_preset("qwen3-ksa-tiny").merge({
        "num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64, "intermediate_dim": 128, "vocab_size": 256,
        "head_dim": 16, "num_heads": 4, "num_kv_heads": 2, "summary_chunk_size": chunk,
        "summary_sliding_chunk_num": window, "summary_token_num": n_sum, "summary_token_begin": 200})


def _build(cfg):
    torch.manual_seed(0)
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    return model.float()


def _worker(rank, world, port, L, chunk, window, n_sum, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ksa_b200.parallel.cp import CpContext, shard_inputs
        cfg = _cfg(chunk, window, n_sum)
        model = _build(cfg)
        B = 2
        g = torch.Generator().manual_seed(3)
        toks = torch.randint(0, 200, (B, L + 1), generator=g)
        tokens, labels = shard_inputs(toks[:, :-1], toks[:, 1:], rank, world)
        model.cp = CpContext(dist.group.WORLD, L, chunk, n_sum, cfg.num_kv_heads, cfg.head_dim, batch=B,
                             n_heads=cfg.num_heads)
        loss = model(tokens, labels)
        loss.backward()
        grads = {n: p.grad.numpy().copy() for n, p in model.named_parameters() if p.grad is not None}
        hidden = model(tokens, return_hidden=True).detach().numpy()
        out_q.put((rank, float(loss.detach()), grads, hidden))   # numpy: pickled by value, not by shared handle
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L,chunk,window,n_sum", [(2, 128, 16, 2, 1), (4, 128, 16, 3, 2)])
def test_context_parallel_model_matches_whole_sequence(world, L, chunk, window, n_sum):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, L, chunk, window, n_sum, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q.get(timeout=240) for _ in range(world)], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    cfg = _cfg(chunk, window, n_sum)
    model = _build(cfg)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 200, (2, L + 1), generator=g)
    loss = model(toks[:, :-1].contiguous(), toks[:, 1:].contiguous())
    loss.backward()
    hidden = model(toks[:, :-1].contiguous(), return_hidden=True).detach()
    # equal token counts per shard: the mean of the shard losses is the whole-sequence loss
    assert abs(sum(r[1] for r in results) / world - float(loss.detach())) < 1e-5
    Ll = L // world
    for r, _, _, h in results:
        torch.testing.assert_close(torch.from_numpy(h), hidden[:, r * Ll:(r + 1) * Ll], atol=2e-5, rtol=1e-4)
    for n, p in model.named_parameters():
        if p.grad is None:
            continue
        avg = torch.from_numpy(sum(r[2][n] for r in results) / world)
        torch.testing.assert_close(avg, p.grad, atol=2e-5, rtol=1e-3, msg=lambda m: f"{n}: {m}")


def test_halo_sources_cover_window_across_owners():
    from ksa_b200.parallel.cp import CpContext, CpShape
    sh = CpShape(rank=3, size=4, seq_len=512, chunk=16, n_sum=1)
    assert sh.local_len == 128 and sh.local_sum == 8
    assert sh.halo_len(2) == 32 and sh.halo_len(None) == 384 and sh.halo_len(20) == 320
    cp = CpContext.__new__(CpContext)
    cp.rank, cp.size, cp.shape = 3, 4, sh
    assert cp.text_sources(32) == [(2, 96, 32)]
    assert cp.text_sources(320) == [(0, 64, 64), (1, 0, 128), (2, 0, 128)]
    assert CpShape(0, 4, 512, 16, 1).halo_len(8) == 0


def test_recipe_runs_with_context_parallel_ranks(tmp_path):
    """The pre-training recipe on two gloo ranks with --context-parallel-size 2: each rank trains on its half of every
    sequence and the run finishes with matching step counts."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = _cfg(16, 2, 1)
    mc = tmp_path / "model.json"
    cfg.save(str(mc))
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen(
            [sys.executable, os.path.join(root, "recipes", "pretrain_ksa.py"), "--model-config", str(mc), "--output-dir",
             str(tmp_path / "out"), "--max-length", "128", "--seed", "1", "--model-dtype", "float32", "--learning-rate",
             "1e-3", "--lr-scheduler-type", "constant", "--num-training-steps", "3", "--context-parallel-size", "2",
             "--comm", "collective", "--logging-per-step", "1", "--heartbeat-timeout", "30"],
            env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs[0][-2000:]
    done = json.loads([l for l in outs[0].splitlines() if l.startswith('{"done"')][-1])
    assert done["steps"] == 3 and done["loss"] is not None and done["loss"] < 7.0
