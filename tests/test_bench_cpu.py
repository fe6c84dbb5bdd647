"""Host-side checks of bench.py that need no GPU: the CPU (reference-semantics) arm prints one JSON
line with the contract's keys, and the tensor-parallel planning helpers behave."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("workload,metric", [("gemm", "w8a8_gemm_tops"), ("norm", "dq_add_layernorm_q_gbytes_per_s"),
                                             ("opt1.3b", "int8_opt_prefill_tokens_per_s")])
def test_reference_arm_prints_one_json_line(workload, metric):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", workload,
                          "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == metric and d["value"] > 0
    for key in ("unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "config", "cpu_baseline", "e2e"):
        assert key in d
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"]


def test_reference_arm_does_not_load_the_product():
    """The CPU arm must map neither the product package nor its CUDA library, and its `config` is the one
    the repository's own arm reports for the same workload."""
    code = ("import runpy, sys, json, io, contextlib\n"
            "sys.argv = ['bench.py', '--impl', 'reference', '--workload', 'opt1.3b', '--steps', '1', '--warmup', '1']\n"
            "buf = io.StringIO()\n"
            "with contextlib.redirect_stdout(buf):\n"
            "    mod = runpy.run_path('bench.py', run_name='__main__')\n"
            "assert not any(m == 'torch_int' or m.startswith('torch_int.') for m in sys.modules), 'product imported'\n"
            "maps = open('/proc/self/maps').read()\n"
            "assert 'libtorch_int_b200' not in maps, 'product library mapped'\n"
            "line = json.loads(buf.getvalue().strip())\n"
            "assert line['config'] == mod['opt_config_dict']('opt1.3b', 1), line['config']\n"
            "assert '512-token sequence' in line['cpu_baseline']['sample']\n")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]


def test_reference_arm_other_ranks_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_pipeline_planning():
    from torch_int.models.tensor_parallel import TensorParallel
    tp = TensorParallel(8, 3, max_chunks=4)
    assert tp.plan_chunks(16, 1024) == 4          # whole sequences per group, rows divisible by the ranks
    assert tp.plan_chunks(16, 1) == 0             # decode steps: one all-reduce per exchange instead
    assert tp.plan_chunks(3, 1024) == 3 and tp.plan_chunks(5, 1000) == 1 and tp.plan_chunks(2, 77 * 4) == 0
    assert TensorParallel(2, 0).plan_chunks(2, 77) == 0
    tp.min_pipeline_tokens = 32
    assert tp.plan_chunks(4, 48) == 4 and tp.plan_chunks(2, 77) == 0


def test_peer_workspace_addressing():
    """Slab and row arithmetic of the peer-memory exchange (no GPU: fields filled by hand)."""
    from torch_int.models.tensor_parallel import PeerWorkspace, TensorParallel
    ws = object.__new__(PeerWorkspace)
    ws.tp = TensorParallel(4, 2)
    ws.chunks, ws.mc, ws.ms, ws.e = 3, 64, 16, 32
    ws.stage_off, ws.h8_off = 0, 3 * 4 * 16 * 32 * 4
    ws.ptrs = [1 << 40, 2 << 40, 3 << 40, 4 << 40]
    sc = ws.scatter_ptrs(1)
    # my (rank 2) slab of chunk 1 in every owner's stage: ((c * n + rank) * ms * e) int32 elements in
    assert sc == [p + ((1 * 4 + 2) * 16 * 32) * 4 for p in ws.ptrs]
    assert ws.q_dst_ptrs(2) == [p + ws.h8_off + 2 * 64 * 32 for p in ws.ptrs]
    # slabs of different ranks and chunks never overlap and stay inside the stage area
    seen = set()
    for r in range(4):
        ws.tp = TensorParallel(4, r)
        for c in range(3):
            start = ws.scatter_ptrs(c)[0] - ws.ptrs[0]
            assert start % (16 * 32 * 4) == 0 and start + 16 * 32 * 4 <= ws.h8_off
            assert start not in seen
            seen.add(start)


def test_stream_trace_bookkeeping():
    """StreamTrace with injected events: spans land on their rows with the right offsets and durations,
    and the summary adds up (the real events are CUDA events; only the arithmetic is checked here)."""
    from torch_int.models.tensor_parallel import StreamTrace, TensorParallel

    class Clock:
        now = 0.0

    class Event:
        def record(self, stream):
            self.t = Clock.now

        def elapsed_time(self, other):      # milliseconds, like torch.cuda.Event
            return other.t - self.t

    tr = StreamTrace(new_event=Event)
    tp = TensorParallel(2, 0)
    assert tp.trace is None
    with tp.span("ignored", "compute", None):      # tracing off: a no-op context
        Clock.now += 5.0
    tp.trace = tr
    Clock.now = 10.0
    with tp.span("gemm", "compute", None, group=0):
        Clock.now += 2.0
    with tp.span("push", "exchange", None, group=0):
        Clock.now += 0.5
    with tp.span("gemm", "compute", None, group=1):
        Clock.now += 1.0
    ev = [e for e in tr.events(pid=3) if e["ph"] == "X"]
    assert [(e["name"], e["tid"], round(e["ts"]), round(e["dur"])) for e in ev] == [
        ("gemm", 0, 0, 2000), ("push", 1, 2000, 500), ("gemm", 0, 2500, 1000)]
    assert all(e["pid"] == 3 for e in ev) and ev[0]["args"] == {"group": 0}
    names = {e["tid"]: e["args"]["name"] for e in tr.events() if e["ph"] == "M"}
    assert names == {0: "compute", 1: "exchange"}
    s = tr.summary()
    assert round(s["compute"]["busy_us"]) == 3000 and round(s["compute"]["last_us"]) == 3500
    assert round(s["exchange"]["by_name"]["push"]) == 500
