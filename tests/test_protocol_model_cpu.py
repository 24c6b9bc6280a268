"""The kernel's scheduling protocol on CPU "ranks" (tests/protocol_model/protocol_model.cpp:
std::atomic state machines, one host thread per CTA, one control block per rank).

What the GPU tests cannot show without faulting or hanging a GPU is shown here: every
attention task, O_proj slot and AllReduce slot runs exactly once over several launches with
no reset in between; the control words are zero after every launch; and when a message is
lost, a rank is late, or a rank has left between two steps, the bounded waits report a
status and every thread returns (the reference's waits are unbounded:
fused_fa_oproj_ar.py:90-95, 137-142, 263-268)."""
import json
import os
import subprocess

import pytest

SRC = os.path.join(os.path.dirname(__file__), "protocol_model", "protocol_model.cpp")


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("pm") / "protocol_model")
    subprocess.run(["g++", "-O2", "-std=c++17", "-pthread", SRC, "-o", exe], check=True)

    def run(*args, timeout=60):
        res = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=timeout)
        assert res.returncode == 0, res.stderr
        return json.loads(res.stdout)
    return run


@pytest.mark.parametrize("tp,ctas,tiles,heads,nsg", [(1, 5, 9, 4, 3), (2, 6, 12, 4, 3),
                                                     (4, 4, 10, 2, 5), (8, 3, 7, 2, 4)])
def test_every_task_runs_exactly_once_and_the_exit_is_clean(model, tp, ctas, tiles, heads, nsg):
    out = model("--tp", tp, "--ctas", ctas, "--tiles", tiles, "--heads", heads, "--nsg", nsg,
                "--launches", 6, "--limit-ms", 5000)
    assert out["launches_ok"] == 6 and out["exactly_once"] and out["clean_exit"], out
    assert all(s == [0, 0] for s in out["status"]), out


@pytest.mark.parametrize("pairing,heads", [(1, 4), (1, 8), (2, 2), (2, 3), (2, 5), (2, 8)])
def test_attention_tasks_of_two_heads_count_every_head_once(model, pairing, heads):
    """The kernel's two-head attention tasks: heads sharing a kv head (the counter steps by
    two over head ids) and heads that share none (the counter numbers tasks, the last head of
    an odd count runs alone).  Every (row tile, head) once, the row tile's head count reaches
    H exactly once, six launches without a reset."""
    out = model("--tp", 2, "--ctas", 5, "--tiles", 9, "--heads", heads, "--nsg", 3,
                "--pairing", pairing, "--launches", 6, "--limit-ms", 5000)
    assert out["launches_ok"] == 6 and out["exactly_once"] and out["clean_exit"], out
    assert all(s == [0, 0] for s in out["status"]), out


def test_a_straggler_rank_is_waited_for(model):
    out = model("--tp", 3, "--launches", 3, "--straggler", 1, 60, "--limit-ms", 3000)
    assert out["launches_ok"] == 3 and out["exactly_once"] and out["clean_exit"], out


def test_a_lost_arrival_ends_in_statuses_not_in_a_hang(model):
    # rank 1 never reports slot 4 (owner: rank 4 % 2 = 0): rank 0 runs out of work with one
    # owned slot never ready (idle time-out, code 6); rank 1 finishes and times out in the
    # rank barrier (code 4) because rank 0 left without signalling
    out = model("--tp", 2, "--launches", 3, "--drop-arrival", 1, 4, "--limit-ms", 200)
    assert out["launches_ok"] == 0, out
    assert out["status"][0][0] == 6 and out["status"][1][0] == 4, out
    assert out["worst_launch_ms"] < 5000, out


def test_a_rank_that_left_between_steps_times_the_others_out(model):
    out = model("--tp", 3, "--launches", 4, "--leave", 2, 2, "--limit-ms", 200)
    assert out["launches_ok"] == 2 and out["exactly_once"] and out["clean_exit"], out
    assert out["status"][0][0] != 0 and out["status"][1][0] != 0 and out["status"][2][0] == 0, out
    assert out["worst_launch_ms"] < 5000, out
