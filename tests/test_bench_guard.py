"""The part of ``bench.py`` that runs after the headline measurement (the mixture-of-experts measurement
reported under ``"secondary"``, then the tear-down) must never cost the headline line: an exception there is
recorded, a hang is ended by a deadline that prints the line and exits with code 0. Exercised on the CPU with
stand-ins for the measurement."""
import json
import os
import subprocess
import sys
import textwrap

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(body: str, timeout_s: str = "2", world: int = 2, rank: int = 0):
    script = textwrap.dedent(f"""
        import sys, time
        sys.path.insert(0, {REPO!r})
        import bench
        from types import SimpleNamespace
        args = SimpleNamespace(steps=5, warmup=3)
        line = {{"metric": "m", "value": 1.0}} if {rank} == 0 else None
        teardown = lambda: None
    """) + textwrap.dedent(body) + textwrap.dedent(f"""
        bench.finish_with_secondary(args, line, {rank}, {world}, None, False, teardown)
    """)
    env = dict(os.environ, PICO_BENCH_SECONDARY_TIMEOUT=timeout_s)
    return subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=120, env=env)


def _lines(out):
    return [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]


def test_secondary_result_is_attached_to_the_one_line():
    out = _run("bench.measure_config = lambda a, ref: {'value': 7.0, 'steps': a.steps, 'config': a.config}\n", "30")
    assert out.returncode == 0, out.stderr
    (line,) = _lines(out)
    assert line["value"] == 1.0 and line["secondary"] == {"value": 7.0, "steps": 3, "config": "moe"}


def test_an_exception_in_the_secondary_part_is_recorded():
    out = _run("def boom(a, ref):\n    raise RuntimeError('no such kernel')\nbench.measure_config = boom\n", "30")
    assert out.returncode == 0, out.stderr
    (line,) = _lines(out)
    assert line["value"] == 1.0 and "RuntimeError: no such kernel" in line["secondary"]["unavailable"]


def test_a_hanging_secondary_part_ends_at_the_deadline_with_the_headline_printed():
    out = _run("bench.measure_config = lambda a, ref: time.sleep(60)\n", "1")
    assert out.returncode == 0, out.stderr
    (line,) = _lines(out)
    assert line["value"] == 1.0 and "not finished" in line["secondary"]["unavailable"]


def test_a_hanging_teardown_prints_nothing_twice():
    out = _run("bench.measure_config = lambda a, ref: {'value': 2.0}\nteardown = lambda: time.sleep(60)\n", "2")
    assert out.returncode == 0, out.stderr
    (line,) = _lines(out)
    assert line["secondary"] == {"value": 2.0}


def test_other_ranks_exit_quietly_at_the_deadline():
    out = _run("bench.measure_config = lambda a, ref: time.sleep(60)\n", "1", rank=1)
    assert out.returncode == 0 and _lines(out) == []


def test_one_gpu_has_no_secondary_part():
    out = _run("def never(a, ref):\n    raise AssertionError('must not run')\nbench.measure_config = never\n", "30", world=1)
    assert out.returncode == 0, out.stderr
    (line,) = _lines(out)
    assert line == {"metric": "m", "value": 1.0}


def test_a_failing_or_hanging_release_keeps_the_headline():
    for rel, timeout, needle in (("def bad():\n    raise RuntimeError('close failed')\n", "30", "release failed: RuntimeError: close failed"),
                                 ("def bad():\n    time.sleep(60)\n", "1", "not finished")):
        script = textwrap.dedent(f"""
            import sys, time
            sys.path.insert(0, {REPO!r})
            import bench
            from types import SimpleNamespace
            args = SimpleNamespace(steps=5, warmup=3)
            line = {{"metric": "m", "value": 1.0}}
            def never(a, ref):
                raise AssertionError("the secondary part must not run after a failed release")
            bench.measure_config = never
        """) + rel + "bench.finish_with_secondary(args, line, 0, 2, None, False, lambda: None, bad)\n"
        out = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=120,
                             env=dict(os.environ, PICO_BENCH_SECONDARY_TIMEOUT=timeout))
        assert out.returncode == 0, out.stderr
        (got,) = _lines(out)
        assert got["value"] == 1.0 and needle in got["secondary"]["unavailable"], got

