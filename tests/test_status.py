"""The device status word: how a kernel's bounded wait that ran out reaches the caller.

CPU tests drive the host-side read-back with a stand-in for the device state; the GPU test runs the
library's own probe kernel, whose wait is meant to run out (nothing faults or hangs)."""
import types

import pytest
import torch

from xattn_b200 import _native


class _FakeEvent:
    def __init__(self, done):
        self.done = done

    def query(self):
        return self.done


def _fake_state(value, done=True):
    return types.SimpleNamespace(sm_count=148, status=torch.tensor([value], dtype=torch.int32),
                                 host=torch.tensor([value], dtype=torch.int32), event=_FakeEvent(done))


def test_raise_status_names_site_and_code():
    with pytest.raises(RuntimeError, match=r"status 1 at wait site 80"):
        _native._raise_status((80 << 8) | 1)
    with pytest.raises(RuntimeError, match=r"nondecreasing.*|decrease along batch row 5"):
        _native._raise_status((5 << 8) | 3)


def test_asynchronous_read_back_raises_at_the_next_launch(monkeypatch):
    """A status copied back by an earlier launch is examined before the next one: non-zero raises and
    clears the device word; a read-back still in flight is left alone; zero passes."""
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    dev = torch.device("cuda", 0)
    st = _fake_state((62 << 8) | 1)
    monkeypatch.setattr(_native, "_state", lambda device: st)
    with pytest.raises(RuntimeError, match="wait site 62"):
        _native._pre_launch(dev)
    assert st.event is None and int(st.status[0]) == 0
    pending = _fake_state((62 << 8) | 1, done=False)
    monkeypatch.setattr(_native, "_state", lambda device: pending)
    assert _native._pre_launch(dev) is pending and pending.event is not None
    clean = _fake_state(0)
    monkeypatch.setattr(_native, "_state", lambda device: clean)
    assert _native._pre_launch(dev) is clean and clean.event is None


def test_no_event_queries_during_graph_capture(monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: True)
    st = _fake_state((62 << 8) | 1)
    monkeypatch.setattr(_native, "_state", lambda device: st)
    assert _native._pre_launch(torch.device("cuda", 0)) is st      # looked at after the replay instead
    _native._post_launch(st)
    assert isinstance(st.event, _FakeEvent)


@pytest.mark.gpu
def test_wait_that_runs_out_reports_and_leaves_the_context_usable(cuda_device, monkeypatch):
    import xattn_b200 as xattn
    xattn.check_status()
    monkeypatch.setattr(_native, "_SYNC_CHECK", False)          # asynchronous path: raise at the next check
    _native.selftest_wait_timeout(cuda_device, budget_us=2000)
    with pytest.raises(RuntimeError, match=r"status 1 at wait site 99"):
        xattn.check_status()
    xattn.check_status()                                        # the word was cleared
    monkeypatch.setattr(_native, "_SYNC_CHECK", True)           # synchronous path: raise at the launch itself
    with pytest.raises(RuntimeError, match=r"wait site 99"):
        _native.selftest_wait_timeout(cuda_device, budget_us=500)
    # the context still works
    q = torch.randn(1, 64, 2, 64, device=cuda_device, dtype=torch.bfloat16)
    y, _ = xattn.causal_flash_attn_fwd(q, q[:, :, :1], q[:, :, :1])
    xattn.check_status()
    assert torch.isfinite(y).all()


@pytest.mark.gpu
def test_unsorted_key_ids_are_reported(cuda_device):
    """Key segment ids that decrease along a row break the plan's binary search: the plan kernels say so."""
    import xattn_b200 as xattn
    q = torch.randn(2, 256, 2, 64, device=cuda_device, dtype=torch.bfloat16)
    ids = (torch.arange(256, device=cuda_device) // 100).expand(2, -1).contiguous()
    xattn.causal_flash_attn_fwd(q, q, q, segment_idx=ids)
    xattn.check_status()
    bad = ids.clone()
    bad[1, 130] = 0                                             # 1 1 1 0 1 ... in batch row 1
    with pytest.raises(RuntimeError, match="batch row 1"):
        xattn.causal_flash_attn_fwd(q, q, q, segment_idx=bad)
        xattn.check_status()
    xattn.check_status()
