"""Process groups and the Ulysses primitives on gloo ranks (world 4, context-parallel size 2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ksa_b200.parallel import groups as G
        G.initialize_model_parallel(2)
        # contiguous CP blocks, strided DP groups; data is shared within a CP group
        assert G.get_context_parallel_world_size() == 2 and G.get_data_parallel_world_size() == 2
        assert G.get_context_parallel_rank() == rank % 2 and G.get_data_parallel_rank() == rank // 2
        assert G.get_context_parallel_ranks() == [rank - rank % 2, rank - rank % 2 + 1]
        cpg, cpr = G.get_context_parallel_group(), G.get_context_parallel_rank()
        # batch broadcast inside the CP group, then label pre-shifting split
        batch = {"input_ids": torch.arange(16)[None] + 100 * rank, "note": "kept"}
        G.broadcast_batch_tensors(batch)
        assert int(batch["input_ids"][0, 0]) == 100 * (rank - rank % 2)
        full = batch["input_ids"].clone()
        part = G.split_batch_for_context_parallel(dict(batch), cpr, 2)
        assert part["input_ids"].shape == (1, 8) and torch.equal(part["input_ids"][0], full[0, cpr * 8:cpr * 8 + 8])
        want = torch.cat([full[0, 1:], torch.tensor([-100])])[cpr * 8:cpr * 8 + 8]
        assert torch.equal(part["labels"][0], want)          # a shard's last label is its successor's first token
        # Ulysses: sequence-sharded [B, S/P, H, D] -> head-sharded [B, S, H/P, D] and back, with gradients
        B, S, H, D = 2, 6, 4, 3
        gen = torch.Generator().manual_seed(7 + rank // 2)
        whole = torch.randn(B, S, H, D, generator=gen)
        local = whole[:, cpr * 3:(cpr + 1) * 3].clone().requires_grad_(True)
        heads = G.SeqAllToAll4D.apply(cpg, local, 2, 1)
        assert heads.shape == (B, S, H // 2, D)
        assert torch.allclose(heads, whole[:, :, cpr * 2:(cpr + 1) * 2])
        back = G.SeqAllToAll4D.apply(cpg, heads, 1, 2)
        assert torch.allclose(back, local)
        (back * torch.arange(D)).sum().backward()
        assert torch.allclose(local.grad, torch.arange(D).float().expand_as(local))
        # autograd all-gather along the sequence
        x = whole[:, cpr * 3:(cpr + 1) * 3].clone().requires_grad_(True)
        gathered = G.AllGather.apply(x, 1, cpg)
        assert torch.allclose(gathered, whole)
        (gathered * 2).sum().backward()
        assert torch.allclose(x.grad, torch.full_like(x, 2.0 * 2))      # every rank of the group contributes
        assert torch.allclose(G.gather_by_group(x.detach(), cpg, dim=1), whole)
        G.destroy_model_parallel()
        out_q.put((rank, "ok"))
    except Exception:
        import traceback
        out_q.put((rank, traceback.format_exc()[-2000:]))
    finally:
        dist.destroy_process_group()


def test_groups_and_ulysses_primitives_on_four_ranks():
    world = 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r, status in res:
        assert status == "ok", f"rank {r}: {status}"


def test_node_topology_from_the_launcher_environment(monkeypatch):
    """Peer memory ends at the node: the helpers that decide between the fused and the collective back ends read the
    launcher's environment (torchrun or Open MPI)."""
    from ksa_b200.parallel import groups
    for k in ("WORLD_SIZE", "LOCAL_WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_SIZE"):
        monkeypatch.delenv(k, raising=False)
    assert groups.local_world_size() == 1 and not groups.spans_nodes()
    assert groups.local_world_size(8) == 8 and not groups.spans_nodes(8)            # nothing said: one node
    monkeypatch.setenv("WORLD_SIZE", "16")
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    assert groups.local_world_size() == 8 and groups.spans_nodes() and groups.spans_nodes(16)
    groups.check_context_parallel_placement(1)
    groups.check_context_parallel_placement(4)
    groups.check_context_parallel_placement(8)
    for bad in (16, 3):
        with pytest.raises(ValueError):
            groups.check_context_parallel_placement(bad)
    monkeypatch.delenv("LOCAL_WORLD_SIZE")
    monkeypatch.delenv("WORLD_SIZE")
    monkeypatch.setenv("OMPI_COMM_WORLD_SIZE", "32")
    monkeypatch.setenv("OMPI_COMM_WORLD_LOCAL_SIZE", "8")
    assert groups.local_world_size() == 8 and groups.spans_nodes()
    monkeypatch.setenv("OMPI_COMM_WORLD_LOCAL_SIZE", "32")
    assert not groups.spans_nodes()
    # variables left over from another launch (a test runner started under a 1-process launcher spawns 2 ranks)
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "1")
    assert groups.local_world_size(2) == 2 and not groups.spans_nodes(2)
