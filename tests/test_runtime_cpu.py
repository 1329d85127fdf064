"""Host-side logic of the symmetric-memory runtime that needs no GPU: the epoch bookkeeping that lets
a captured CUDA graph be replayed (kernels take epochs relative to a device-side base word that the
graph's last node advances), checked against a small model of the device; and the reference's import
paths served by this package."""
import importlib

import pytest


class _FakeDevice:
    """What the kernels do with epochs: absolute epoch = base[slot] + relative epoch."""

    def __init__(self):
        self.base = {}
        self.seen = []          # (slot, absolute epoch) in launch order

    def launch(self, slot, rel):
        self.seen.append((slot, self.base.get(slot, 0) + rel))

    def add_base(self, slots, deltas):
        for s, d in zip(slots, deltas):
            self.base[s] = self.base.get(s, 0) + d


def _group(dev, monkeypatch):
    from picotron_b200.runtime import symm
    g = symm.SymmGroup.__new__(symm.SymmGroup)
    g._epochs = [0] * symm.FLAG_SLOTS
    g._base = [0] * symm.FLAG_SLOTS
    g._recording = None
    g.flags = type("F", (), {"local_ptr": 0})()
    fake_ext = type("E", (), {"epoch_base_add": staticmethod(lambda ptr, slots, deltas: dev.add_base(slots, deltas))})
    monkeypatch.setattr(symm.ops, "ext", lambda: fake_ext)
    monkeypatch.setattr(symm.ops, "count_launch", lambda n=1: None)
    return g


def test_graph_replays_continue_the_epoch_count(monkeypatch):
    dev = _FakeDevice()
    g = _group(dev, monkeypatch)
    # eager use before any capture
    for _ in range(3):
        dev.launch(0, g.next_epoch(0))
    # capture: two uses of slot 0, one of slot 5; nothing executes while capturing
    g.begin_graph()
    captured = [(0, g.next_epoch(0)), (0, g.next_epoch(0)), (5, g.next_epoch(5))]
    rec = g.end_graph()              # in a real capture the base advance is recorded as the last node
    dev.base = {}                    # ... so it has not run yet
    assert rec.used == {0: 2, 5: 1}

    def replay():
        rec.before_replay()
        for slot, rel in captured:
            dev.launch(slot, rel)
        dev.add_base(list(rec.used), list(rec.used.values()))
        rec.after_replay()

    replay()
    replay()
    dev.launch(0, g.next_epoch(0))   # an eager launch on a slot the graph uses
    dev.launch(7, g.next_epoch(7))   # and on one it does not
    replay()
    dev.launch(5, g.next_epoch(5))
    per_slot = {}
    for slot, e in dev.seen:
        per_slot.setdefault(slot, []).append(e)
    for slot, es in per_slot.items():
        assert es == list(range(1, len(es) + 1)), (slot, es)     # every slot counts 1, 2, 3, ... without gaps
    assert len(per_slot[0]) == 3 + 2 * 3 + 1 and len(per_slot[5]) == 3 + 1 and per_slot[7] == [1]


def test_reference_import_paths_are_served():
    pairs = {
        "picotron.process_group_manager": "picotron_b200.process_group_manager",
        "picotron.model": "picotron_b200.models.llama",
        "picotron.tensor_parallel.tensor_parallel": "picotron_b200.parallel.tensor_parallel",
        "picotron.pipeline_parallel.pp_schedules": "picotron_b200.parallel.pp_schedules",
        "picotron.expert_parallel.expert_parallel": "picotron_b200.parallel.expert_parallel",
        "picotron.data_parallel.zero": "picotron_b200.parallel.zero",
        "picotron.utils": "picotron_b200.utils",
    }
    for alias, target in pairs.items():
        assert importlib.import_module(alias) is importlib.import_module(target), alias
    from picotron.context_parallel.context_parallel import apply_context_parallel, ring_attention  # noqa: F401
    from picotron.tensor_parallel.tp_communications import vocab_parallel_cross_entropy  # noqa: F401
    import picotron.process_group_manager as pgm
    import picotron_b200.process_group_manager as ours
    marker = object()
    old = ours.process_group_manager
    try:
        pgm.process_group_manager = marker               # module state is shared, not copied
        assert ours.process_group_manager is marker
    finally:
        ours.process_group_manager = old


@pytest.mark.parametrize("world", [2, 4])
def test_protocol_model_finds_no_race_in_the_fused_tp_protocol(world):
    """Random interleavings of ranks and streams over the operation list of the fused tensor-parallel
    path: two alternating copies of each buffer, pushes on a communication stream, with and without
    kept gather buffers (which need the barrier that opens a micro-batch)."""
    from picotron_b200.runtime.protocol_model import build_program, simulate
    for keep in (False, True):
        prog = build_program(layers=3, micro_batches=3, keep_gathered=keep, barrier=keep)
        for seed in range(25):
            assert simulate(world, prog, seed) == [], (keep, seed)
    # pushes on the main stream (PICO_TP_COMM_STREAM=0) are the same protocol with less freedom
    prog = build_program(layers=2, micro_batches=2, keep_gathered=False, barrier=False, comm_stream=False)
    for seed in range(10):
        assert simulate(world, prog, seed) == []


def test_protocol_model_detects_the_races_the_design_rules_out():
    """The model has teeth: drop a rule and some schedule shows the race it prevents."""
    from picotron_b200.runtime.protocol_model import build_program, simulate

    def races(**kw):
        prog = build_program(layers=2, micro_batches=3, **kw)
        return any(simulate(3, prog, seed) for seed in range(60))

    assert races(keep_gathered=True, barrier=False), \
        "kept gather buffers without the barrier at the start of a micro-batch must race"
    assert races(keep_gathered=False, barrier=False, double_buffer=False), \
        "a single copy of the gather / staging buffers must race"
    assert not races(keep_gathered=True, barrier=True)


@pytest.mark.parametrize("world", [2, 4])
def test_protocol_model_finds_no_race_in_the_expert_exchanges(world):
    """The exchanges of a mixture-of-experts layer (expert-load rows, dispatch, combine, and their backward
    counterparts): no schedule reads a block before it arrived or after it was overwritten. Because the
    kinds of exchange strictly alternate, that holds even on one copy per slab; the second copy is what
    makes two exchanges of one kind in a row safe (two token tiles dispatched back to back), and the model
    shows the race without it."""
    from picotron_b200.runtime.protocol_model import build_moe_program, simulate
    for prog in (build_moe_program(layers=3, micro_batches=3), build_moe_program(layers=2, micro_batches=2, load_sum=False),
                 build_moe_program(layers=2, micro_batches=2, double_buffer=False)):
        for seed in range(20):
            assert simulate(world, prog, seed) == [], seed
    tiled = dict(layers=2, micro_batches=2, tiles=2)
    assert not any(simulate(world, build_moe_program(**tiled), seed) for seed in range(20))
    assert any(simulate(world, build_moe_program(double_buffer=False, **tiled), seed) for seed in range(60)), \
        "two dispatches in a row on a single copy of the slab must race"


def test_flat_params_switch_follows_zero_stage():
    """``training.flat_params``: unset = flat buffers unless ZeRO stage 2/3 asks for sharded gradients and
    parameters (the per-parameter wrappers); an explicit value wins."""
    from types import SimpleNamespace
    from picotron_b200.engine import TrainEngine

    def wanted(flat, stage):
        stub = SimpleNamespace(cfg={"training": {"flat_params": flat}, "distributed": {"zero_stage": stage}},
                               pgm=SimpleNamespace(global_rank=1))
        return TrainEngine._flat_wanted(stub)

    assert [wanted(None, s) for s in (0, 1, 2, 3)] == [True, True, False, False]
    assert wanted(True, 3) is True and wanted(False, 0) is False


def test_race_jitter_is_off_by_default_and_seeded_per_rank(monkeypatch):
    from picotron_b200.runtime import symm
    monkeypatch.delenv("PICO_RACE_JITTER", raising=False)
    assert symm._Jitter().rng is None
    monkeypatch.setenv("PICO_RACE_JITTER", "5")
    a, b = symm._Jitter(), symm._Jitter()
    assert a.rng is not None and [a.rng.randrange(1000) for _ in range(4)] == [b.rng.randrange(1000) for _ in range(4)]
    a()      # no GPU, no capture: a call is a no-op
