"""Tensor-parallel inference on CPU ranks (gloo): sharded prefill + decode equal the unsharded engine."""
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


def _cfg(tied: bool):
    return get_preset("qwen3-ksa-tiny").merge({
        "num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64, "intermediate_dim": 128, "vocab_size": 256,
        "head_dim": 16, "num_heads": 4, "num_kv_heads": 2, "summary_chunk_size": 8, "summary_sliding_chunk_num": 2,
        "summary_token_num": 1, "summary_token_begin": 200, "tie_word_embeddings": tied})


def _full_model(cfg):
    torch.manual_seed(0)
    model = get_model_class(cfg.model_class)(cfg)
    model.init_weights(seed=0)
    return model.float()


def _run_engine(model, prompt, steps):
    from ksa_b200.inference.engine import KsaInferenceEngine
    eng = KsaInferenceEngine(model, max_len=64, batch=prompt.shape[0])
    outs = [eng.prefill(prompt)]
    nxt = outs[0].argmax(-1)
    for _ in range(steps):
        outs.append(eng.decode_step(nxt))
        nxt = outs[-1].argmax(-1)
    return torch.stack(outs)


def _worker(rank, world, port, tied, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ksa_b200.parallel.tp import TpContext, build_tp_model
        cfg = _cfg(tied)
        full = _full_model(cfg)
        tp = TpContext(dist.group.WORLD, cfg.embed_dim, max_rows=256)
        model = build_tp_model(full.state_dict(), cfg, tp)
        assert model.config.num_heads == cfg.num_heads // world
        g = torch.Generator().manual_seed(5)
        prompt = torch.randint(0, 200, (2, 21), generator=g)
        out_q.put((rank, _run_engine(model, prompt, 12).numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tied", [False, True])
def test_tensor_parallel_engine_matches_single_rank(tied):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tied, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q.get(timeout=240) for _ in range(world)], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    cfg = _cfg(tied)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 200, (2, 21), generator=g)
    ref = _run_engine(_full_model(cfg), prompt, 12)
    for _, out in results:
        torch.testing.assert_close(torch.from_numpy(out), ref, atol=1e-4, rtol=1e-4)


def test_shard_state_dict_partitions_every_projection():
    from ksa_b200.parallel.tp import shard_state_dict, tp_local_config
    cfg = _cfg(False)
    full = _full_model(cfg).state_dict()
    shards = [shard_state_dict(full, cfg, r, 2) for r in range(2)]
    Hq, Hkv, Dh, F = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.intermediate_dim
    w = full["layers.0.attn.wqkv.weight"]
    q = torch.cat([s["layers.0.attn.wqkv.weight"][:Hq // 2 * Dh] for s in shards])
    assert torch.equal(q, w[:Hq * Dh])
    o = torch.cat([s["layers.0.attn.output_proj.weight"] for s in shards], dim=1)
    assert torch.equal(o, full["layers.0.attn.output_proj.weight"])
    w2 = torch.cat([s["layers.1.mlp.w2.weight"] for s in shards], dim=1)
    assert torch.equal(w2, full["layers.1.mlp.w2.weight"])
    head = torch.cat([s["output.weight"] for s in shards])
    assert torch.equal(head, full["output.weight"])
    local = tp_local_config(cfg, 2)
    assert (local.num_heads, local.num_kv_heads, local.intermediate_dim) == (Hq // 2, Hkv // 2, F // 2)
    with pytest.raises(ValueError):
        tp_local_config(cfg, 3)
