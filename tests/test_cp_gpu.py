"""Context parallelism on 2 and 4 GPUs: halo / summary exchange over peer memory against the whole-sequence kernels.
Each case is skipped on a box with fewer GPUs than ranks."""
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


def _shard_rows(B, L, Ns, r, P, dev):
    Ll, Nsl = L // P, Ns // P
    text = (torch.arange(B, device=dev)[:, None] * L + r * Ll + torch.arange(Ll, device=dev)[None, :]).reshape(-1)
    if Ns == 0:
        return text
    summ = (B * L + torch.arange(B, device=dev)[:, None] * Ns + r * Nsl + torch.arange(Nsl, device=dev)[None, :]).reshape(-1)
    return torch.cat([text, summ])


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from ksa_b200 import ops
        from ksa_b200.ops import _lib
        from ksa_b200.parallel.cp import CpContext, cp_attention_packed, shard_inputs
        dev = torch.device("cuda", rank)
        # head counts that divide by the group size, so that the heads-resharded full layers apply
        B, L, C, S, W, Hq, Hkv, D = 2, 2048, 128, 1, 3, 2 * world, world, 128
        Ns = (L // C) * S
        g = torch.Generator(device="cpu").manual_seed(5)
        cps = {m: CpContext(dist.group.WORLD, L, C, S, Hkv, D, batch=B, device=dev, full_layers=True, n_heads=Hq,
                            full_layer_mode=m) for m in ("halo", "ulysses")}
        # summary layers, then full layers staged (halo) and resharded to heads (ulysses); the last pass reuses slots
        for summaries, mode in ((True, "halo"), (False, "halo"), (False, "ulysses"), (True, "ulysses"), (False, "ulysses")):
            cp = cps[mode]
            ns = Ns if summaries else 0
            full = (torch.randn(B * (L + ns), (Hq + 2 * Hkv) * D, generator=g) * 0.5).to(dev).bfloat16()
            go = torch.randn(B * (L + ns), Hq * D, generator=g).to(dev).bfloat16()
            rows = _shard_rows(B, L, ns, rank, world, dev)
            x_full = full.clone().requires_grad_(True)
            if summaries:
                o_full = ops.attention_packed(x_full, B, L, ns, Hq, Hkv, D, C, S, W)
            else:
                o_full = ops.attention_packed(x_full, B, L, 0, Hq, Hkv, D)
            o_full.backward(go)
            x_loc = full[rows].clone().requires_grad_(True)
            o_loc = cp_attention_packed(x_loc, cp, Hq, Hkv, D, W if summaries else None, summaries)
            o_loc.backward(go[rows])
            torch.cuda.synchronize(); _lib.check_status(); dist.barrier()
            torch.testing.assert_close(o_loc.float(), o_full[rows].float(), atol=2e-2, rtol=2e-2)
            ref_g = x_full.grad[rows].float()
            err = (x_loc.grad.float() - ref_g).norm() / ref_g.norm()
            assert err < 2e-2, (summaries, mode, float(err))
        for c in cps.values():
            c.close()

        # summary layers with the exchange inside the attention kernels: tile-aligned shapes (256 summaries and a
        # 128-key halo per rank); five layers in a row so that every exchange slot and return block is reused
        from ksa_b200.parallel.cp import direct_exchange_possible
        B, L, C, S, W = 2, 4096, 8, 1, 16
        Ns = (L // C) * S
        cp = CpContext(dist.group.WORLD, L, C, S, Hkv, D, batch=B, device=dev, max_window=W, n_heads=Hq)
        names = []
        real_call = _lib.call
        _lib.call = lambda name, *a: (names.append(name), real_call(name, *a))[1]
        try:
            for it in range(5):
                full = (torch.randn(B * (L + Ns), (Hq + 2 * Hkv) * D, generator=g) * 0.5).to(dev).bfloat16()
                go = torch.randn(B * (L + Ns), Hq * D, generator=g).to(dev).bfloat16()
                rows = _shard_rows(B, L, Ns, rank, world, dev)
                x_full = full.clone().requires_grad_(True)
                o_full = ops.attention_packed(x_full, B, L, Ns, Hq, Hkv, D, C, S, W)
                o_full.backward(go)
                x_loc = full[rows].clone().requires_grad_(True)
                assert direct_exchange_possible(cp, x_loc, D, W)
                o_loc = cp_attention_packed(x_loc, cp, Hq, Hkv, D, W, True)
                o_loc.backward(go[rows])
                torch.cuda.synchronize(); _lib.check_status(); dist.barrier()
                torch.testing.assert_close(o_loc.float(), o_full[rows].float(), atol=2e-2, rtol=2e-2)
                ref_g = x_full.grad[rows].float()
                err = (x_loc.grad.float() - ref_g).norm() / ref_g.norm()
                assert err < 2e-2, ("direct", it, float(err))
        finally:
            _lib.call = real_call
        assert "ksa_attn_fwd_cp" in names and "ksa_attn_bwd_fused_cp" in names
        assert not any(n in ("ksa_peer_copy", "ksa_peer_add_bf16") for n in names), sorted(set(names))
        cp.close()

        # whole model: shard loss / gradients against the whole sequence on one GPU
        from ksa_b200.config import get_preset
        from ksa_b200.models import get_model_class
        cfg = get_preset("qwen3-ksa-tiny").merge({"head_dim": 128, "num_heads": 2 * world, "num_kv_heads": world,
                                                  "embed_dim": 512,
                                                  "summary_chunk_size": 128, "summary_sliding_chunk_num": 2,
                                                  "num_layers": 2, "summary_layer_freq": [1, 0]})
        torch.manual_seed(0)
        model = get_model_class(cfg.model_class)(cfg)
        model.init_weights(seed=0)
        model = model.to(dev).to(torch.bfloat16)
        Lm = 1024
        toks = torch.randint(0, cfg.vocab_size, (1, Lm + 1), generator=g).to(dev)
        loss_full = model(toks[:, :-1].contiguous(), toks[:, 1:].contiguous())
        loss_full.backward()
        ref_grads = {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None}
        tokens, labels = shard_inputs(toks[:, :-1], toks[:, 1:], rank, world)
        for mode in ("halo", "ulysses"):
            model.zero_grad(set_to_none=True)
            model.cp = CpContext(dist.group.WORLD, Lm, 128, cfg.summary_token_num, cfg.num_kv_heads, cfg.head_dim, batch=1,
                                 device=dev, full_layers=True, n_heads=cfg.num_heads, full_layer_mode=mode)
            loss = model(tokens, labels)
            loss.backward()
            torch.cuda.synchronize(); _lib.check_status()
            lsum = loss.detach().float().clone()
            dist.all_reduce(lsum)
            assert abs(float(lsum) / world - float(loss_full)) < 3e-2, (float(lsum) / world, float(loss_full))
            for n, p in model.named_parameters():
                if p.grad is None:
                    continue
                gsum = p.grad.float().clone()
                dist.all_reduce(gsum)
                gsum /= world
                err = (gsum - ref_grads[n]).norm() / ref_grads[n].norm().clamp_min(1e-6)
                assert err < 5e-2, (mode, n, float(err))
            model.cp.close()
            model.cp = None
        out_q.put((rank, "ok"))
    except Exception as exc:  # report instead of leaving the parent to time out
        import traceback
        out_q.put((rank, "error: " + "".join(traceback.format_exception(exc))[-3000:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_context_parallel_attention_and_model(world):
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
