"""What bench.py answers without a GPU: more than one GPU is refused with exit code 2 and one line, the reference
arm says in one JSON line why it is unavailable and exits 0; the planner of untimed steps; the timeline writer."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def run(*argv):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *argv], capture_output=True, text=True, timeout=120)
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    return p.returncode, lines


def test_more_than_one_gpu_is_refused_with_one_line():
    rc, lines = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert rc == 2 and len(lines) == 1
    assert json.loads(lines[0])["n_gpus"] == 2


def test_reference_arm_says_why_it_is_unavailable():
    rc, lines = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert rc == 0 and len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_timed_window_lies_in_the_middle_of_the_growth():
    # few timed steps: they end at the middle of the growth from the prompt to the last context
    assert bench.untimed_steps(256, 3, 2048, 4096) == 1024 - 256
    # a window longer than half the growth is centred on it; never fewer untimed steps than the warm-up
    assert bench.untimed_steps(2000, 3, 2048, 4096) == 24
    assert bench.untimed_steps(2048, 8, 2048, 4096) == 8


def test_timeline_writer_sums_by_kernel(tmp_path):
    def launch(name, blocks, begin, waited, end):
        return SimpleNamespace(name=name, blocks=blocks, begin_us=begin, waited_us=waited, end_us=end, ctas=[])
    launches = [launch("a", 4, 0.0, 0.5, 2.0), launch("b", 8, 1.5, 2.0, 5.0), launch("a", 4, 4.0, 5.0, 6.0)]
    out = tmp_path / "t.md"
    import fellm_b200.engine.timeline as timeline
    old = (timeline.Timeline.phases, timeline.Timeline.table)
    timeline.Timeline.phases = staticmethod(lambda ls: "(phases)")
    timeline.Timeline.table = staticmethod(lambda ls: "(table)")
    try:
        total = bench.write_timeline(str(out), "three launches", launches)
    finally:
        timeline.Timeline.phases, timeline.Timeline.table = old
    assert total == 6.0
    text = out.read_text()
    assert text.startswith("three launches: 3 launches, 6.0 us")
    # kernel a: two launches, 1.5 + 1.0 us of run, 0.5 + 1.0 before their waits, one gap of -1.0 (4.0 - 5.0)
    assert "| a | 4 | 2 | 1.25 | 0.75 | -0.50 | 3.0 |" in text
    assert "| b | 8 | 1 | 3.00 | 0.50 | -0.50 | 3.0 |" in text
