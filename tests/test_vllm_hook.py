"""The vLLM hook's dispatch logic with a stand-in GroupCoordinator (no GPU, no vLLM import):
pass-through for world size 1, everything the library cannot take goes to the original method
and is counted as a fallback (reference: step3b/vllm_tp_bench.py:87-126)."""
import torch

from libtbvcoll_b200.integrations import vllm_hook, dbo_patch


class FakeGroup:
    def __init__(self, world, name):
        self.world_size, self.unique_name, self.rank_in_group = world, name, 0
        self.orig_calls = 0

    def all_reduce(self, x):
        self.orig_calls += 1
        return x + 100

    def _all_reduce_out_place(self, x):
        self.orig_calls += 1
        return x + 200


def test_hook_falls_back_and_counts():
    vllm_hook.uninstall()
    vllm_hook.stats.update(calls=0, fallbacks=0, wrapper_s=0.0)
    vllm_hook.install(group_coordinator_cls=FakeGroup)
    try:
        vllm_hook._state["tp_name"] = "tp:0"
        single = FakeGroup(1, "tp:0")
        x = torch.ones(4)
        assert single.all_reduce(x) is x and single.orig_calls == 0            # world size 1: untouched
        other = FakeGroup(2, "pp:0")
        assert torch.equal(other.all_reduce(x), x + 100) and other.orig_calls == 1   # not the TP group
        tp = FakeGroup(2, "tp:0")
        vllm_hook._state["raw"], vllm_hook._state["cap"] = (lambda *a: -2), 1 << 20  # library declines everything
        assert torch.equal(tp.all_reduce(x), x + 100)                          # CPU tensor -> fallback
        assert torch.equal(tp._all_reduce_out_place(x), x + 200)               # the compiled-graph door is wrapped too
        assert torch.equal(tp.all_reduce(torch.ones(4, dtype=torch.int32)), torch.ones(4, dtype=torch.int32) + 100)
        # tracing placeholders (FakeTensor): must never reach the native call, whatever the library says
        from torch._subclasses.fake_tensor import FakeTensorMode
        called = []
        vllm_hook._state["raw"] = lambda *a: called.append(a) or 0
        with FakeTensorMode():
            fake = torch.empty(8, dtype=torch.bfloat16)
            tp.all_reduce(fake)
        assert called == []
        vllm_hook._state["raw"] = (lambda *a: -2)
        assert vllm_hook.stats["calls"] == 4 and vllm_hook.stats["fallbacks"] == 4
        assert "fallbacks" in vllm_hook.summary()
    finally:
        vllm_hook.uninstall()
    assert FakeGroup(2, "tp:0").all_reduce(torch.zeros(1)).item() == 100       # original restored


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
