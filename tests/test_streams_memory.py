"""Stream pool / SM split set-up and device memory queries against stand-ins for the driver, the extension and NVML
(reference: "kv-cache pipeline"/nanovllm/utils/streams.py:17-123, nanovllm/utils/memory.py:6-18)."""
import sys
import types

import pytest
import torch

from fastcache_b200.utils import memory, streams


class _Stream:
    def __init__(self, handle, device=None):
        self.cuda_stream = handle
        self.device = device


class _Ext:
    """The extension's green-context entry points: 148 SMs, partitions in groups of 4."""

    def __init__(self, fail=False):
        self.fail, self.created, self.extra, self.registered = fail, [], [], {}
        self._next = 1000

    def sm_count(self, index):
        return 148

    def greenctx_create(self, index, want, a, b):
        if self.fail:
            raise RuntimeError("driver says no")
        self.created.append((index, want))
        comp = -(-want // 4) * 4
        self._next += 10
        main, first = self._next, self._next + 1
        self._next += 1
        return {"main_stream": main, "compress_stream": first, "main_sms": 148 - comp,
                "compress_sms": comp, "total_sms": 148}

    def greenctx_extra_stream(self, base, flags):
        self._next += 1
        self.extra.append(base)
        return self._next

    def register_stream_sms(self, handle, sms):
        self.registered[handle] = sms


@pytest.fixture
def fake_ext(monkeypatch):
    from fastcache_b200.ops import loader
    ext = _Ext()
    monkeypatch.setattr(loader, "ext", lambda: ext)
    monkeypatch.setattr(loader, "ext_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "ExternalStream", _Stream)
    monkeypatch.setattr(streams, "_PARTITIONS", {})
    return ext


def test_split_is_created_once_per_size_and_streams_know_their_sms(fake_ext):
    dev = torch.device("cuda", 0)
    got = streams.try_create_greenctx_streams(dev, 36 / 148, n_compress=2)
    assert fake_ext.created == [(0, 36)]
    assert (got["main_sms"], got["compress_sms"], got["total_sms"]) == (112, 36, 148)
    assert len(got["compress"]) == 2 and got["compress"][0].cuda_stream != got["compress"][1].cuda_stream
    assert fake_ext.registered[got["main"].cuda_stream] == 112
    assert all(fake_ext.registered[s.cuda_stream] == 36 for s in got["compress"])
    # the same split again: nothing new is created; a third stream is added to the cached partition
    again = streams.try_create_greenctx_streams(dev, 36 / 148, n_compress=3)
    assert fake_ext.created == [(0, 36)] and len(again["compress"]) == 3
    assert again["main"] is got["main"] and again["compress"][:2] == got["compress"]
    assert fake_ext.registered[again["compress"][2].cuda_stream] == 36
    fewer = streams.try_create_greenctx_streams(dev, 36 / 148, n_compress=1)
    assert len(fewer["compress"]) == 1 and fake_ext.created == [(0, 36)]
    # another size is another partition; the driver's rounding shows in the SM counts
    other = streams.try_create_greenctx_streams(dev, 0.5, n_compress=1)
    assert fake_ext.created == [(0, 36), (0, 74)] and other["compress_sms"] == 76 and other["main_sms"] == 72


def test_refusal_by_the_driver_is_a_fallback_not_an_error(fake_ext, capsys, monkeypatch):
    fake_ext.fail = True
    assert streams.try_create_greenctx_streams(torch.device("cuda", 0), 0.25) is None
    assert "green contexts unavailable" in capsys.readouterr().out
    from fastcache_b200.ops import loader
    monkeypatch.setattr(loader, "ext_available", lambda: False)          # no extension at all
    assert streams.try_create_greenctx_streams(torch.device("cuda", 0), 0.25) is None


def test_stream_pool_round_robin_and_info():
    pool = streams.StreamPool("main", ["a", "b", "c"], True, {"compress_sms": 36})
    assert [pool.next_stream() for _ in range(5)] == ["a", "b", "c", "a", "b"]
    assert pool.streams == ["a", "b", "c"] and pool.greenctx_info.available
    plain = streams.StreamPool("main", ["a"], False, {"fallback": "priority"})
    info = plain.greenctx_info
    assert not info.available and info.reason == "priority"
    assert streams.StreamPool("m", [], False, {}).greenctx_info.reason == "not requested"
    cpu = streams.build_streams(torch.device("cpu"), n_compress=2, use_greenctx=True)
    assert cpu.main is None and cpu.compress == [] and not cpu.greenctx and cpu.next_stream() is None


def test_memory_query_without_a_device_and_through_nvml(monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert memory.get_gpu_memory() == (0, 0, 0)
    # a device is visible: torch's numbers by default
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 1)
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda d: (30 << 30, 180 << 30))
    assert memory.get_gpu_memory() == (180 << 30, 150 << 30, 30 << 30)
    # NVML on request: the index goes through CUDA_VISIBLE_DEVICES (visible device 1 is physical GPU 5)
    asked = []
    nvml = types.ModuleType("pynvml")
    nvml.nvmlInit = lambda: None
    nvml.nvmlDeviceGetHandleByIndex = lambda i: asked.append(i) or ("handle", i)
    nvml.nvmlDeviceGetMemoryInfo = lambda h: types.SimpleNamespace(total=100, used=60, free=40)
    monkeypatch.setitem(sys.modules, "pynvml", nvml)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3,5")
    assert memory.get_gpu_memory(use_nvml=True) == (100, 60, 40) and asked == [5]
    # NVML that fails falls back to torch's numbers
    nvml.nvmlInit = lambda: (_ for _ in ()).throw(RuntimeError("no NVML"))
    assert memory.get_gpu_memory(1, use_nvml=True) == (180 << 30, 150 << 30, 30 << 30)
