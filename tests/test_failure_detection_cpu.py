"""Failure detection without touching a GPU: failures are made on the host (a rank that raises or exits, a stalled
step, a damaged checkpoint) and the survivors must stop cleanly or recover."""
import json
import os
import shutil
import socket
import subprocess
import sys
import time

import pytest
import torch
import torch.distributed as dist

from ksa_b200.config import get_preset
from ksa_b200.utils.watchdog import FaultInjector, HeartbeatMonitor, RankFailure, StepWatchdog

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_watchdog_reports_a_stalled_step_once():
    seen = []
    with StepWatchdog(0.15, on_timeout=seen.append, poll_s=0.02) as wd:
        for _ in range(5):
            time.sleep(0.05)
            wd.beat()
        assert not seen
        time.sleep(0.4)
    assert len(seen) == 1 and seen[0] > 0.15 and wd.fired


def test_heartbeat_monitor_sees_abort_records_missing_ranks_and_rendezvous():
    store = dist.HashStore()
    a = HeartbeatMonitor(store, 0, 2, timeout_s=0.2)
    b = HeartbeatMonitor(store, 1, 2, timeout_s=0.2)
    a.check(); b.check()
    # both arrive: agree returns
    import threading
    t = threading.Thread(target=lambda: b.agree(1))
    t.start(); a.agree(1); t.join()
    # rank 1 reports a failure instead of arriving: rank 0 stops at the rendezvous, nothing launched
    b.report_failure("boom")
    with pytest.raises(RankFailure, match="rank 1 reported: boom"):
        a.agree(2)
    # a rank that silently stops beating is found after the timeout
    c = HeartbeatMonitor(dist.HashStore(), 0, 2, timeout_s=0.1)
    time.sleep(0.25)
    with pytest.raises(RankFailure, match="never sent a heartbeat"):
        c.check(); time.sleep(0.15); c.check()
    with pytest.raises(RankFailure, match="not every rank arrived"):
        c.agree(5)


def test_fault_injector_spec():
    fi = FaultInjector("raise@step=3,rank=1; stall@step=1,rank=1,seconds=0.01", rank=1)
    fi.at_step(0); fi.at_step(1)
    with pytest.raises(RuntimeError, match="injected failure on rank 1 at step 3"):
        fi.at_step(3)
    FaultInjector("raise@step=3,rank=1", rank=0).at_step(3)
    with pytest.raises(ValueError):
        FaultInjector("explode@step=1")


def _launch(rank, world, port, args, env_extra):
    env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
               MASTER_PORT=str(port), PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", **env_extra)
    return subprocess.Popen([sys.executable, os.path.join(ROOT, "recipes", "pretrain_ksa.py")] + args, env=env,
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


def _model_json(tmp_path):
    cfg = get_preset("qwen3-ksa-tiny").merge({"num_layers": 2, "summary_layer_freq": [1, 0], "embed_dim": 64,
                                               "intermediate_dim": 128, "vocab_size": 256, "summary_token_begin": 256,
                                               "head_dim": 16, "summary_chunk_size": 16})
    mc = tmp_path / "model.json"
    cfg.save(str(mc))
    return str(mc)


@pytest.mark.parametrize("kind", ["raise", "exit"])
def test_surviving_rank_stops_between_steps_when_a_peer_fails(tmp_path, kind):
    """Rank 1 fails on the host before step 3; rank 0 must leave the loop with RankFailure within the heartbeat limit
    instead of blocking in the next collective, and a restart from ``latest`` continues the run."""
    out = tmp_path / "run"
    base = ["--model-config", _model_json(tmp_path), "--output-dir", str(out), "--max-length", "64", "--seed", "1",
            "--model-dtype", "float32", "--learning-rate", "1e-3", "--lr-scheduler-type", "constant",
            "--save-checkpoint-per-step", "2", "--num-training-steps", "6", "--heartbeat-timeout", "6",
            "--comm", "collective"]
    port = _free_port()
    procs = [_launch(r, 2, port, base, {"KSA_FAULT": f"{kind}@step=3,rank=1"}) for r in range(2)]
    t0 = time.time()
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert time.time() - t0 < 200
    assert procs[1].returncode != 0
    assert procs[0].returncode != 0 and "RankFailure" in outs[0], outs[0][-2000:]
    assert (out / "latest").read_text() == "global_step2"
    # recovery: same command, no fault, resume from latest
    port = _free_port()
    procs = [_launch(r, 2, port, base + ["--checkpoint-dir", str(out), "--resume-weights", "--resume-optimizer"], {})
             for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs[0][-2000:]
    assert (out / "latest").read_text() == "global_step6"


def test_resume_falls_back_over_a_damaged_checkpoint(tmp_path):
    from recipes.pretrain_ksa import get_argument_parser, train
    out = tmp_path / "run"
    base = ["--model-config", _model_json(tmp_path), "--output-dir", str(out), "--max-length", "64", "--seed", "1",
            "--model-dtype", "float32", "--learning-rate", "1e-3", "--lr-scheduler-type", "constant",
            "--save-checkpoint-per-step", "2"]
    train(get_argument_parser().parse_args(base + ["--num-training-steps", "4"]))
    assert (out / "latest").read_text() == "global_step4"
    # a crash during the save of step 4: its metadata never got written
    os.remove(out / "global_step4" / ".metadata")
    resume = base + ["--num-training-steps", "6", "--checkpoint-dir", str(out), "--resume-weights", "--resume-optimizer"]
    from torch.distributed.checkpoint.api import CheckpointException
    with pytest.raises((Exception, CheckpointException)):
        train(get_argument_parser().parse_args(resume))
    r = train(get_argument_parser().parse_args(resume + ["--resume-fallback"]))
    assert r["steps"] == 6          # resumed from step 2, ran 4 more
    # a truncated dataloader state is ignored, not fatal
    from ksa_b200.training import checkpoint as ckpt
    (out / "global_step2" / "dataloader_state.pt").write_bytes(b"\x00\x01")

    class _DS:
        def load_state_dict(self, s):
            raise AssertionError("must not be reached")
    assert ckpt.load_dataloader_state(_DS(), str(out / "global_step2")) is False


def test_checkpoint_survives_a_change_of_world_size(tmp_path):
    """Saved by two FSDP ranks, resumed by one process, saved again and resumed by two ranks (the step counter,
    optimizer state and LR schedule go on)."""
    from recipes.pretrain_ksa import get_argument_parser, train
    out = tmp_path / "run"
    base = ["--model-config", _model_json(tmp_path), "--output-dir", str(out), "--max-length", "64", "--seed", "1",
            "--model-dtype", "float32", "--learning-rate", "1e-3", "--lr-scheduler-type", "constant",
            "--save-checkpoint-per-step", "2", "--comm", "collective"]
    port = _free_port()
    # the two ranks keep their optimizer state in host memory (--cpu-offload): the shards are saved from there
    procs = [_launch(r, 2, port, base + ["--num-training-steps", "4", "--heartbeat-timeout", "30", "--cpu-offload"], {})
             for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs[0][-2000:]
    assert (out / "latest").read_text() == "global_step4"
    # every rank wrote its own rows only: two data files of about the same size, and the metadata records each
    # parameter as two row chunks
    files = sorted(f for f in os.listdir(out / "global_step4") if f.endswith(".distcp"))
    sizes = [sum(os.path.getsize(out / "global_step4" / f) for f in files if f.startswith(f"__{r}_")) for r in (0, 1)]
    assert min(sizes) > 0.8 * max(sizes), (files, sizes)
    import torch.distributed.checkpoint as dcp
    meta = dcp.FileSystemReader(str(out / "global_step4")).read_metadata()
    chunks = meta.state_dict_metadata["app.model.model.layers.0.mlp.w2.weight"].chunks
    assert len(chunks) == 2 and chunks[0].sizes[0] == chunks[1].sizes[0] and chunks[1].offsets[0] == chunks[0].sizes[0]
    # the single-process reader of the converters puts the row chunks back together
    from ksa_b200.training.checkpoint import dcp_to_state_dict
    from ksa_b200.tools.convert import flatten_model_state
    tree = flatten_model_state(dcp_to_state_dict(str(out / "global_step4")))
    assert tree["model.layers.0.mlp.w2.weight"].shape[0] == 2 * chunks[0].sizes[0]
    r = train(get_argument_parser().parse_args(base + ["--num-training-steps", "6", "--checkpoint-dir", str(out),
                                                        "--resume-weights", "--resume-optimizer", "--logging-per-step", "1"]))
    assert r["steps"] == 6 and r["loss"] is not None and r["loss"] < 6.5
    assert (out / "latest").read_text() == "global_step6"
    # and back: the single process's checkpoint resumed by two ranks
    port = _free_port()
    procs = [_launch(r, 2, port, base + ["--num-training-steps", "8", "--checkpoint-dir", str(out), "--resume-weights",
                                         "--resume-optimizer", "--heartbeat-timeout", "30"], {}) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs[0][-2000:]
    assert (out / "latest").read_text() == "global_step8"
