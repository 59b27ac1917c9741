"""The vLLM hook's dispatch logic with a stand-in GroupCoordinator (no GPU, no vLLM import):
pass-through for world size 1, everything the library cannot take goes to the original method
and is counted as a fallback (reference: step3b/vllm_tp_bench.py:87-126)."""
import torch

from libtbvcoll_b200.integrations import vllm_hook, dbo_patch


class FakeGroup:
    """Current vLLM: all_reduce forwards (through a custom op) to _all_reduce_out_place."""
    def __init__(self, world, name):
        self.world_size, self.unique_name, self.rank_in_group = world, name, 0
        self.orig_calls = 0

    def all_reduce(self, x):
        if self.world_size == 1:
            return x
        return self._all_reduce_out_place(x)

    def _all_reduce_out_place(self, x):
        self.orig_calls += 1
        return x + 200


class OldFakeGroup:
    """A vLLM without the out-of-place door: all_reduce is the only method (what the reference patches)."""
    def __init__(self, world, name):
        self.world_size, self.unique_name, self.rank_in_group = world, name, 0
        self.orig_calls = 0

    def all_reduce(self, x):
        self.orig_calls += 1
        return x + 100


def _arm(tp_obj, raw, cap=1 << 20):
    """Stand in for an initialised library: bind the fast path to a fake C function."""
    from libtbvcoll_b200 import tbvcoll
    vllm_hook._state["tp"] = tp_obj
    old = (tbvcoll.raw_fn, tbvcoll.cap)
    tbvcoll.raw_fn, tbvcoll.cap = (lambda: raw), (lambda: cap)
    try:
        vllm_hook._bind_fast()
    finally:
        tbvcoll.raw_fn, tbvcoll.cap = old
    vllm_hook._state["world"] = tp_obj.world_size


def test_hook_wraps_the_single_runtime_door_and_counts_fallbacks():
    vllm_hook.uninstall()
    vllm_hook.stats.update(calls=0, fallbacks=0, wrapper_s=0.0)
    orig_all_reduce = FakeGroup.all_reduce
    vllm_hook.install(group_coordinator_cls=FakeGroup)
    try:
        assert vllm_hook._state["door"] == "_all_reduce_out_place"
        assert FakeGroup.all_reduce is orig_all_reduce                         # the traceable method is left alone
        tp, other, single = FakeGroup(2, "tp:0"), FakeGroup(2, "pp:0"), FakeGroup(1, "tp:0")
        _arm(tp, lambda *a: -2)                                                # library declines everything
        x = torch.ones(4)
        assert single.all_reduce(x) is x and single.orig_calls == 0            # world size 1: untouched
        assert torch.equal(other.all_reduce(x), x + 200) and other.orig_calls == 1   # not the TP group: original, not counted
        assert vllm_hook.stats["calls"] == 0
        assert torch.equal(tp.all_reduce(x), x + 200)                          # CPU tensor -> fallback
        assert torch.equal(tp.all_reduce(torch.ones(4, dtype=torch.int32)), torch.ones(4, dtype=torch.int32) + 200)
        # tracing placeholders (FakeTensor): must never reach the native call, whatever the library says
        from torch._subclasses.fake_tensor import FakeTensorMode
        called = []
        _arm(tp, lambda *a: called.append(a) or 0)
        with FakeTensorMode():
            fake = torch.empty(8, dtype=torch.bfloat16)
            tp._all_reduce_out_place(fake)
        assert called == []
        assert vllm_hook.stats["calls"] == 3 and vllm_hook.stats["fallbacks"] == 3
        assert "fallbacks" in vllm_hook.summary()
    finally:
        vllm_hook.uninstall()
    assert FakeGroup(2, "tp:0").all_reduce(torch.zeros(1)).item() == 200       # original restored


def test_hook_on_a_vllm_without_the_out_of_place_door():
    vllm_hook.uninstall()
    vllm_hook.stats.update(calls=0, fallbacks=0, wrapper_s=0.0)
    vllm_hook.install(group_coordinator_cls=OldFakeGroup)
    try:
        assert vllm_hook._state["door"] == "all_reduce"
        tp = OldFakeGroup(2, "tp:0")
        _arm(tp, lambda *a: -2)
        x = torch.ones(4)
        assert OldFakeGroup(1, "tp:0").all_reduce(x) is x
        assert torch.equal(tp.all_reduce(x), x + 100) and vllm_hook.stats["fallbacks"] == 1
    finally:
        vllm_hook.uninstall()


def test_eager_install_after_plain_install_and_world_mismatch(monkeypatch):
    """install(eager=True) may follow a plain install() and then brings the library up from the launcher's
    environment (here: a 1-rank world, for which there is nothing to bring up); a TP group whose size differs
    from the world the library was brought up for switches the hook off instead of mixing protocols."""
    vllm_hook.uninstall()
    monkeypatch.setenv("WORLD_SIZE", "1")
    vllm_hook.install(group_coordinator_cls=FakeGroup)
    vllm_hook.install(eager=True, group_coordinator_cls=FakeGroup)             # no early return before the eager part
    try:
        assert vllm_hook._state["installed"] and vllm_hook._state["fast"] is None
        tp = FakeGroup(4, "tp:0")
        _arm(tp, lambda *a: 0)
        vllm_hook._state["world"] = 2                                          # brought up for 2 ranks, TP group has 4
        vllm_hook._state["tp"] = None
        import types, sys
        fake_ps = types.ModuleType("vllm.distributed.parallel_state")
        fake_ps.get_tp_group = lambda: tp
        for name in ("vllm", "vllm.distributed"):
            monkeypatch.setitem(sys.modules, name, sys.modules.get(name) or types.ModuleType(name))
        monkeypatch.setitem(sys.modules, "vllm.distributed.parallel_state", fake_ps)
        x = torch.ones(4)
        assert torch.equal(tp.all_reduce(x), x + 200) and vllm_hook._state["dead"]
        assert torch.equal(tp.all_reduce(x), x + 200) and tp.orig_calls == 2   # and it stays off
    finally:
        vllm_hook.uninstall()


def test_dbo_patch_mechanism(tmp_path, monkeypatch):
    import sys
    mod = tmp_path / "fake_vllm_mod.py"
    mod.write_text("def f():\n    assert False, 'blocked'\n    return 1\n")
    monkeypatch.syspath_prepend(str(tmp_path))
    assert dbo_patch.patch("fake_vllm_mod", "assert False, 'blocked'", "pass", "test")
    assert "pass" in mod.read_text() and (tmp_path / "fake_vllm_mod.py.tbv-orig").exists()
    assert dbo_patch.patch("fake_vllm_mod", "assert False, 'blocked'", "pass", "test")     # idempotent
    assert not dbo_patch.patch("fake_vllm_mod", "no such text", "x", "test")
    assert dbo_patch.unpatch("fake_vllm_mod") and "assert False" in mod.read_text()
    assert isinstance(dbo_patch.survey(), dict)
