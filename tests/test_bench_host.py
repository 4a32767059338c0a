"""Host-side pieces of bench.py that need no GPU: how timed steps are dealt to the captured
graphs, and the work counts the throughput figures are divided by."""
import importlib.util
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    if "bench" in sys.modules:
        return sys.modules["bench"]
    spec = importlib.util.spec_from_file_location("bench", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench"] = mod
    spec.loader.exec_module(mod)
    return mod


class _Graph:
    def __init__(self, name, log):
        self.name, self.log = name, log

    def replay(self):
        self.log.append(self.name)


def _runner(variants, log):
    bench = _bench()
    run = bench.GraphRunner(lambda i: log.append(("direct", i)), variants, False)   # no capture without a GPU
    run.graphs = [_Graph(("single", i), log) for i in range(variants)]
    size = min(run.GROUP, variants)
    run.groups = {first: (_Graph(("group", first), log), size) for first in range(0, variants - size + 1, size)} if size > 1 else {}
    return run


def _steps(log, group):
    out = []
    for kind, first in log:
        out += list(range(first, first + group)) if kind == "group" else [first]
    return out


def test_every_step_runs_once_and_in_rotation_order():
    for variants in (1, 2, 4, 6, 30):
        for start, count in ((0, 20), (5, 20), (3, 1), (0, 0), (7, 61)):
            log = []
            run = _runner(variants, log)
            run.run_many(start, count)
            want = [(start + i) % variants for i in range(count)]
            assert _steps(log, min(run.GROUP, variants)) == want, (variants, start, count)


def test_whole_groups_come_from_group_graphs():
    log = []
    run = _runner(4, log)
    run.run_many(0, 20)
    assert log == [("group", 0)] * 5
    log.clear()
    run.run_many(2, 8)          # starts in the middle of a rotation: singles until a group boundary
    assert log == [("single", 2), ("single", 3), ("group", 0), ("single", 0), ("single", 1)]


def test_one_variant_has_no_groups():
    log = []
    run = _runner(1, log)
    assert run.groups == {}
    run.run_many(0, 3)
    assert log == [("single", 0)] * 3


def test_direct_mode_calls_the_step():
    bench = _bench()
    log = []
    run = bench.GraphRunner(lambda i: log.append(i), 4, False)
    run.run_many(3, 4)
    assert log == [3, 4, 5, 6] and run.mode == "direct"


def test_attended_pairs():
    bench = _bench()
    assert bench.unit_pairs(0, 8192) == 8192 * 8193 // 2
    assert bench.unit_pairs(0, 32768, 512) == 512 * 513 // 2 + (32768 - 512) * 512
    # a query range that starts inside the sequence counts only its own rows
    assert bench.unit_pairs(16384, 32768, 512) == 16384 * 512
    assert bench.prefill_flops(4, 8192) == 4.0 * 4 * 8 * 256 * (8192 * 8193 // 2)
