"""Fused FSDP communication kernels on 2 and 4 GPUs: P2P gather, reduce-scatter + AdamW, and the whole engine against
the collective (NCCL) back end.  Each case is skipped on a box with fewer GPUs than ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tiny():
    from ksa_b200.config import get_preset
    return get_preset("qwen3-ksa-tiny").merge({"head_dim": 128, "num_heads": 4, "num_kv_heads": 2, "embed_dim": 512,
                                               "summary_chunk_size": 128, "summary_sliding_chunk_num": 2})


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from ksa_b200.models import get_model_class
        from ksa_b200.ops import _lib
        from ksa_b200.parallel.fsdp import FsdpEngine
        from ksa_b200.parallel.symm import SymmetricBuffer
        dev = torch.device("cuda", rank)
        # --- raw kernels: gather
        n = 1 << 20
        sb = SymmetricBuffer(n * 2 * world)
        t = sb.view(torch.bfloat16)
        t.zero_()
        t[rank * n:(rank + 1) * n] = rank + 1
        torch.cuda.synchronize(); dist.barrier()
        _lib.call("ksa_peer_gather", sb.ptr_array, world, rank, n, 2, None, None, 0, 8)
        torch.cuda.synchronize(); _lib.check_status(); dist.barrier()
        expect = torch.arange(1, world + 1, device=dev).repeat_interleave(n).to(torch.bfloat16)
        assert torch.equal(t[:n * world], expect)
        sb.close()
        # --- engine: fused vs collective, same seeds and data
        cfg = _tiny()
        results = {}
        g = torch.Generator().manual_seed(11)
        data = torch.randint(0, cfg.vocab_size, (3, world, 2, 513), generator=g)
        for comm, overlap in (("collective", "stream"), ("fused", "stream"), ("fused", "gemm2")):
            torch.manual_seed(0)
            model = get_model_class(cfg.model_class)(cfg)
            model.init_weights(seed=0)
            model = model.to(dev).to(torch.bfloat16)
            # gemm2: every GEMM of the tiny model may carry the gather of the next unit
            eng = FsdpEngine(model, lr=1e-3, weight_decay=0.1, clip_value=1.0, world_size=world, rank=rank, comm=comm,
                             overlap=overlap, pair_gather_min_flops=0.0)
            losses = []
            for s in range(3):
                x = data[s, rank].to(dev)
                losses.append(float(eng.train_step(x[:, :-1].contiguous(), x[:, 1:].contiguous())))
            torch.cuda.synchronize(); _lib.check_status(); dist.barrier()
            if comm == "fused":   # one more forward so that the last update has been gathered everywhere
                eng._write_hyper(); eng._overlap_active = False
                for ui in range(len(eng.units)):
                    eng._gather_now(ui)
                torch.cuda.synchronize(); _lib.check_status(); dist.barrier()
            results[(comm, overlap)] = (losses, [u.compute.float().clone() for u in eng.units], float(eng.grad_norm()))
            if comm == "fused":
                eng.close()
        lc, wc, gc = results[("collective", "stream")]
        for key in (("fused", "stream"), ("fused", "gemm2")):
            lf, wf, gf = results[key]
            assert all(abs(a - b) < 3e-2 for a, b in zip(lc, lf)), (key, lc, lf)
            assert abs(gc - gf) < 0.05 * gc, (key, gc, gf)
            for a, b in zip(wc, wf):
                assert (a - b).norm() <= 1e-2 * a.norm().clamp_min(1e-6), key
        # --- ZeRO-3 storage (shards + slot pool, units re-gathered for backward) against the resident copy
        deep = cfg.merge({"num_layers": 6, "summary_layer_freq": [1, 1, 0, 1, 1, 0]})
        zero3 = {}
        for reshard in (False, True):
            torch.manual_seed(0)
            m = get_model_class(deep.model_class)(deep)
            m.init_weights(seed=0)
            eng = FsdpEngine(m.to(dev).to(torch.bfloat16), lr=1e-3, weight_decay=0.1, clip_value=1.0, world_size=world,
                             rank=rank, comm="fused", overlap="stream", reshard_after_forward=reshard)
            ls = []
            for s in range(3):
                x = data[s, rank].to(dev)
                ls.append(float(eng.train_step(x[:, :-1].contiguous(), x[:, 1:].contiguous())))
            torch.cuda.synchronize(); _lib.check_status(); dist.barrier()
            zero3[reshard] = (ls, torch.cat([u.master.clone() for u in eng.units]), eng.compute_weight_bytes())
            eng.close()
        assert all(abs(a - b) < 2e-2 for a, b in zip(zero3[False][0], zero3[True][0])), zero3
        assert (zero3[False][1] - zero3[True][1]).norm() <= 2e-3 * zero3[False][1].norm()
        # --- resume: 2 steps, state out, a NEW engine (fresh flags, step counter moved forward by the load), step 3
        def fresh():
            torch.manual_seed(0)
            m = get_model_class(cfg.model_class)(cfg)
            m.init_weights(seed=0)
            return FsdpEngine(m.to(dev).to(torch.bfloat16), lr=1e-3, weight_decay=0.1, clip_value=1.0,
                              world_size=world, rank=rank, comm="fused", overlap="stream")
        eng = fresh()
        for s in range(2):
            x = data[s, rank].to(dev)
            eng.train_step(x[:, :-1].contiguous(), x[:, 1:].contiguous())
        torch.cuda.synchronize(); _lib.check_status(); dist.barrier()
        state = {"step": eng.step_count,
                 "units": {k: {kk: (vv.clone() if torch.is_tensor(vv) else vv) for kk, vv in u.items()}
                           for k, u in eng.state_dict()["units"].items()}}
        eng.close()
        eng = fresh()
        eng.load_state_dict(state)
        assert eng.step_count == 2
        x = data[2, rank].to(dev)
        resumed = float(eng.train_step(x[:, :-1].contiguous(), x[:, 1:].contiguous()))
        torch.cuda.synchronize(); _lib.check_status(); dist.barrier()
        eng.close()
        uninterrupted = results[("fused", "stream")][0][2]
        assert abs(resumed - uninterrupted) < 3e-2, (resumed, uninterrupted)
        out_q.put((rank, "ok", lf))
    except Exception as e:  # noqa: BLE001
        import traceback
        out_q.put((rank, "fail", traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fused_fsdp_matches_collective(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
    for rank, status, info in res:
        assert status == "ok", f"rank {rank}: {info}"
