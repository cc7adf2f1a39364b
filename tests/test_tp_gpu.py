"""Tensor-parallel inference on 2 and 4 GPUs: fused all-reduce + add + RMSNorm kernel and the sharded engine against
the unsharded one.  Each case is skipped on a box with fewer GPUs than ranks."""
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


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from ksa_b200 import ops
        from ksa_b200.config import get_preset
        from ksa_b200.inference.engine import KsaInferenceEngine
        from ksa_b200.models import get_model_class
        from ksa_b200.ops import _lib, reference as ref
        from ksa_b200.parallel.tp import TpContext, build_tp_model
        dev = torch.device("cuda", rank)
        # --- the fused kernel alone: partial sums of known values, more residual rows than delta rows
        D, rows_x, rows_d = 512, 300, 260
        g = torch.Generator().manual_seed(3)
        x = torch.randn(rows_x, D, generator=g).to(dev).bfloat16()
        parts = [torch.randn(rows_d, D, generator=g).to(dev).bfloat16() for _ in range(world)]
        w = (1 + 0.1 * torch.randn(D, generator=g)).to(dev).bfloat16()
        total = sum(p.float() for p in parts)
        pad = torch.cat([total, total.new_zeros(rows_x - rows_d, D)])
        res_ref, y_ref = ref.add_rms_norm(x.float(), pad, w.float(), 1e-6)
        # one-shot form, then the two-phase form (reduce-scatter of a row shard + gather), forced on for 2 ranks
        for kw in ({}, {"two_phase_rows": 256, "two_phase_min_size": 2}):
            tp = TpContext(dist.group.WORLD, D, max_rows=4096, device=dev, **kw)
            assert bool(tp.two_phase_rows) == (bool(kw) or world >= 3)    # groups of 3 and more default to it
            for it in range(3):   # three calls: both slots and a slot reuse
                res, y = tp.add_rms_norm(x, parts[rank], w, 1e-6)
                torch.cuda.synchronize(); _lib.check_status()
                torch.testing.assert_close(res.float(), res_ref, atol=3e-2, rtol=2e-2)
                torch.testing.assert_close(y.float(), y_ref, atol=3e-2, rtol=2e-2)
            # chained use: the residual output of one call is the input of the next (in place for the two-phase form)
            res2, _ = tp.add_rms_norm(res, parts[rank], w, 1e-6)
            torch.cuda.synchronize(); _lib.check_status()
            res2_ref, _ = ref.add_rms_norm(res_ref.bfloat16().float(), pad, w.float(), 1e-6)
            torch.testing.assert_close(res2.float(), res2_ref, atol=6e-2, rtol=3e-2)
            tp.close()
        # --- two-phase form with the gather of the normalised rows inside the projection that consumes them
        tp = TpContext(dist.group.WORLD, D, max_rows=4096, device=dev, two_phase_rows=256, two_phase_min_size=2,
                       fused_gather=True)
        assert tp.fused_gather
        wc = (0.05 * torch.randn(384, D, generator=g)).to(dev).bfloat16()
        proj_ref = y_ref.bfloat16().float() @ wc.float().t()
        for it in range(3):
            res, y = tp.add_rms_norm(x, parts[rank], w, 1e-6, defer_gather=True)
            proj = tp.col_parallel_linear(y, wc)                  # all-gather -> GEMM in one launch
            tp.flush()                                            # residual rows (side stream) joined
            torch.cuda.synchronize(); _lib.check_status()
            torch.testing.assert_close(proj.float(), proj_ref, atol=6e-2, rtol=3e-2)
            torch.testing.assert_close(res.float(), res_ref, atol=3e-2, rtol=2e-2)
            torch.testing.assert_close(y.float(), y_ref, atol=3e-2, rtol=2e-2)
        res, y = tp.add_rms_norm(x, parts[rank], w, 1e-6, defer_gather=True)
        tp.flush()                                                # nobody took the gather along: flush does it
        torch.cuda.synchronize(); _lib.check_status()
        torch.testing.assert_close(y.float(), y_ref, atol=3e-2, rtol=2e-2)
        res, y = tp.add_rms_norm(x, parts[rank], w, 1e-6, defer_gather=True)
        proj = tp.col_parallel_linear(y[:200], wc)                # fewer rows than were normalised
        res2, _ = tp.add_rms_norm(res, parts[rank], w, 1e-6)      # chained, joins the residual gather by itself
        torch.cuda.synchronize(); _lib.check_status()
        torch.testing.assert_close(proj.float(), proj_ref[:200], atol=6e-2, rtol=3e-2)
        res2_ref, _ = ref.add_rms_norm(res_ref.bfloat16().float(), pad, w.float(), 1e-6)
        torch.testing.assert_close(res2.float(), res2_ref, atol=6e-2, rtol=3e-2)
        tp.close()
        # --- GEMM -> reduce-scatter: the row-parallel GEMM scatters its row blocks into the owners' slots
        acts = [torch.randn(rows_d, 256, generator=g).to(dev).bfloat16() for _ in range(world)]
        wrs = [(0.05 * torch.randn(D, 256, generator=g)).to(dev).bfloat16() for _ in range(world)]
        total2 = sum((acts[r].float() @ wrs[r].float().t()).bfloat16().float() for r in range(world))
        pad2 = torch.cat([total2, total2.new_zeros(rows_x - rows_d, D)])
        res_ref2, y_ref2 = ref.add_rms_norm(x.float(), pad2, w.float(), 1e-6)
        for fused in (False, True):
            tp = TpContext(dist.group.WORLD, D, max_rows=4096, device=dev, two_phase_rows=256, two_phase_min_size=2,
                           push_partials=True, fused_gather=fused)
            assert tp.push_partials
            for it in range(3):
                token = tp.row_parallel_linear(acts[rank], wrs[rank], residual_rows=rows_x)
                res, y = tp.add_rms_norm(x, token, w, 1e-6, defer_gather=fused)
                tp.flush()
                torch.cuda.synchronize(); _lib.check_status()
                torch.testing.assert_close(res.float(), res_ref2, atol=4e-2, rtol=2e-2)
                torch.testing.assert_close(y.float(), y_ref2, atol=4e-2, rtol=2e-2)
            # without the hint the same object falls back to the pulled layout
            partial = tp.row_parallel_linear(acts[rank], wrs[rank])
            res, y = tp.add_rms_norm(x, partial, w, 1e-6)
            torch.cuda.synchronize(); _lib.check_status()
            torch.testing.assert_close(res.float(), res_ref2, atol=4e-2, rtol=2e-2)
            tp.close()
        # --- engine: TP=2 shard against the whole model on the same GPU
        cfg = get_preset("qwen3-ksa-tiny").merge({"head_dim": 128, "num_heads": 2 * world, "num_kv_heads": world,
                                                  "embed_dim": 512,
                                                  "summary_chunk_size": 128, "summary_sliding_chunk_num": 2,
                                                  "num_layers": 2, "summary_layer_freq": [1, 0],
                                                  "intermediate_dim": 1024})
        torch.manual_seed(0)
        full = get_model_class(cfg.model_class)(cfg)
        full.init_weights(seed=0)
        full = full.to(dev).to(torch.bfloat16)
        prompt = torch.randint(0, cfg.vocab_size, (2, 300), generator=g).to(dev)
        steps = 4

        def run(model):
            eng = KsaInferenceEngine(model, max_len=1024, batch=2)
            outs = [eng.prefill(prompt)]
            toks = [ref_toks[0] if ref_toks is not None else outs[0].argmax(-1)]
            for _ in range(steps):
                outs.append(eng.decode_step(toks[-1]))
                toks.append(ref_toks[len(toks)] if ref_toks is not None else outs[-1].argmax(-1))
            return torch.stack(outs), toks
        ref_toks = None
        ref_out, ref_toks = run(full)
        for kw in ({}, {"two_phase_rows": 256, "two_phase_min_size": 2, "fused_gather": True},
                   {"two_phase_rows": 256, "two_phase_min_size": 2, "fused_gather": True,
                    "push_partials": True}):
            tp = TpContext(dist.group.WORLD, cfg.embed_dim, max_rows=2 * (300 + 8), device=dev, **kw)
            model = build_tp_model(full.state_dict(), cfg, tp, device=dev, dtype=torch.bfloat16)
            out, _ = run(model)
            torch.cuda.synchronize(); _lib.check_status()
            err = (out - ref_out).abs().max() / ref_out.abs().max()
            assert err < 4e-2, (kw, float(err))
            tp.close()
        out_q.put((rank, "ok"))
    except Exception as exc:  # report instead of leaving the parent to time out
        import traceback
        out_q.put((rank, "error: " + "".join(traceback.format_exception(exc))[-3000:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_fused_allreduce_and_engine(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in results:
        assert r[1] == "ok", r
