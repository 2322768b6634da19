"""Host-side logic of delta loading, no GPU: the reader of the reference's checkpoint format,
its failure modes, and the background prefetch thread with its pause / abort handshake
(serving/vllm/delta/worker_manager.py:248-376) driven with a fake loader and a fake slot
manager.  Failures are made on the host: missing or truncated files, tensors of the wrong shape,
more deltas than slots, a loader that raises."""
import os
import shutil
import threading
import time
from collections import OrderedDict

import numpy as np
import pytest
import torch

from deltazip_b200.models import DeltaLayerWeights, DeltaModel, SlotLayout, read_reference_tensors
from deltazip_b200.worker_manager import (DeltaRequest, LRUCacheWorkerDeltaManager,
                                          OverlapLRUCacheWorkerDeltaManager, WorkerDeltaManager)
from oracle import deltazip_oracle as O


# ---------------------------------------------------------------------------
# reader of the reference's checkpoint format
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [4, 2])
def test_reference_checkpoint_merge_and_shards(golden_dir, bits):
    """q/k/v and gate/up are concatenated along the output dimension, per rank; o / down are cut
    along the input dimension; unpacking a rank's tensors gives the matching slices of the dense
    deltas the reference's own unpack produced."""
    path = os.path.join(golden_dir, f"ref_ckpt_b{bits}")
    dense = np.load(os.path.join(path, "dense.npz"))
    cfg, full = read_reference_tensors(path)
    assert cfg.bits == bits and cfg.servable()
    assert sorted(full) == ["layers.0.down_proj", "layers.0.gate_up_proj", "layers.0.o_proj",
                            "layers.0.qkv_proj"]

    def unpack(t):
        return O.unpack(t[0].numpy(), t[1].numpy(), t[2].numpy(), bits)

    want_qkv = np.concatenate([dense["self_attn.q_proj"], dense["self_attn.k_proj"],
                               dense["self_attn.v_proj"]])
    assert np.array_equal(unpack(full["layers.0.qkv_proj"]).view(np.uint16), want_qkv.view(np.uint16))
    want_gu = np.concatenate([dense["mlp.gate_proj"], dense["mlp.up_proj"]])
    assert np.array_equal(unpack(full["layers.0.gate_up_proj"]).view(np.uint16), want_gu.view(np.uint16))
    assert np.array_equal(unpack(full["layers.0.down_proj"]).view(np.uint16),
                          dense["mlp.down_proj"].view(np.uint16))
    for rank in range(2):
        _, part = read_reference_tensors(path, tp_rank=rank, tp_size=2)
        h = slice(128 * rank, 128 * (rank + 1))
        i = slice(256 * rank, 256 * (rank + 1))
        want = np.concatenate([dense["self_attn.q_proj"][h], dense["self_attn.k_proj"][h],
                               dense["self_attn.v_proj"][h]])
        assert np.array_equal(unpack(part["layers.0.qkv_proj"]), want)
        assert np.array_equal(unpack(part["layers.0.o_proj"]), dense["self_attn.o_proj"][:, h])
        want = np.concatenate([dense["mlp.gate_proj"][i], dense["mlp.up_proj"][i]])
        assert np.array_equal(unpack(part["layers.0.gate_up_proj"]), want)
        assert np.array_equal(unpack(part["layers.0.down_proj"]), dense["mlp.down_proj"][:, i])


def test_reference_checkpoint_failures(golden_dir, tmp_path):
    src = os.path.join(golden_dir, "ref_ckpt_b4")
    with pytest.raises(FileNotFoundError):
        read_reference_tensors(str(tmp_path / "nowhere"))
    # configuration without the tensor file
    d1 = tmp_path / "no_tensors"
    d1.mkdir()
    shutil.copy(os.path.join(src, "compress_config.json"), d1)
    with pytest.raises(FileNotFoundError):
        read_reference_tensors(str(d1))
    # truncated safetensors file
    d2 = tmp_path / "truncated"
    shutil.copytree(src, d2)
    f = d2 / "deltazip-compressed.safetensors"
    data = f.read_bytes()
    f.write_bytes(data[: len(data) // 3])
    with pytest.raises(Exception) as exc:
        read_reference_tensors(str(d2))
    assert not isinstance(exc.value, (FileNotFoundError, AssertionError))
    # a projection of the wrong shape, a missing projection, an unservable configuration
    from safetensors.torch import load_file, save_file
    state = load_file(os.path.join(src, "deltazip-compressed.safetensors"))
    d3 = tmp_path / "wrong_shape"
    shutil.copytree(src, d3)
    bad = dict(state)
    bad["model.layers.0.self_attn.k_proj.scales"] = bad["model.layers.0.self_attn.k_proj.scales"][:, :100].contiguous()
    save_file(bad, str(d3 / "deltazip-compressed.safetensors"))
    with pytest.raises(ValueError, match="qkv_proj"):
        read_reference_tensors(str(d3))
    d4 = tmp_path / "missing_proj"
    shutil.copytree(src, d4)
    save_file({k: v for k, v in state.items() if ".up_proj." not in k},
              str(d4 / "deltazip-compressed.safetensors"))
    with pytest.raises(ValueError, match="gate_up_proj"):
        read_reference_tensors(str(d4))
    d5 = tmp_path / "dense_delta"
    shutil.copytree(src, d5)
    import json
    cfg = json.loads((d5 / "compress_config.json").read_text())
    cfg["prunen"], cfg["prunem"] = 0, 0
    (d5 / "compress_config.json").write_text(json.dumps(cfg))
    with pytest.raises(ValueError, match="servable"):
        read_reference_tensors(str(d5))


def test_pack_rejects_tensors_that_do_not_fit_the_slot():
    layout = SlotLayout()
    layout.add("layers.0.o_proj", 128, 128, 4)
    ok = DeltaLayerWeights("layers.0.o_proj", qweight=torch.zeros((4, 256), dtype=torch.int32),
                           scales=torch.zeros((1, 128), dtype=torch.float16),
                           meta=torch.zeros((128, 8), dtype=torch.int16))
    arena = DeltaModel(1, 4, {"layers.0.o_proj": ok}).pack(layout)
    assert arena.numel() == layout.total and layout.total % 256 == 0
    bad = DeltaLayerWeights("layers.0.o_proj", qweight=torch.zeros((4, 128), dtype=torch.int32),
                            scales=torch.zeros((1, 128), dtype=torch.float16),
                            meta=torch.zeros((128, 8), dtype=torch.int16))
    with pytest.raises(ValueError, match="qweight"):
        DeltaModel(2, 4, {"layers.0.o_proj": bad}).pack(layout)


# ---------------------------------------------------------------------------
# worker managers with fakes
# ---------------------------------------------------------------------------

class FakeDelta:
    def __init__(self, delta_id):
        self.id = delta_id


class FakeSlotManager:
    """What the worker managers use of DeltaModelManager: a host registry with a capacity (LRU)
    and GPU slots."""

    def __init__(self, capacity=4, delta_slots=2):
        self.capacity, self.delta_slots = capacity, delta_slots
        self.registered = OrderedDict()
        self.active = []
        self.mapping = None

    def __len__(self):
        return len(self.registered)

    def add_delta(self, delta):
        if delta is None:
            raise ValueError("no delta to register (the load failed)")
        if delta.id in self.registered:
            return False
        if len(self.registered) >= self.capacity:
            raise RuntimeError("No free Delta slots.")
        self.registered[delta.id] = delta
        return True

    def get_delta(self, delta_id):
        return self.registered.get(delta_id)

    def list_deltas(self):
        return dict(self.registered)

    def remove_delta(self, delta_id):
        if delta_id in self.active:
            self.active.remove(delta_id)
        return self.registered.pop(delta_id, None) is not None

    def remove_oldest_delta(self):
        return self.remove_delta(next(iter(self.registered)))

    def remove_all_deltas(self):
        self.registered.clear()
        self.active.clear()

    def activate_delta(self, delta_id):
        if delta_id not in self.registered:
            raise KeyError(delta_id)
        if delta_id in self.active:
            return False
        if len(self.active) >= self.delta_slots:
            self.active.pop(0)
        self.active.append(delta_id)
        return True

    def set_delta_mapping(self, mapping):
        self.mapping = mapping


class ScriptedLoader:
    """A loader whose loads can be held at a gate; honours the pause / abort events the way
    DeltaModel.from_checkpoint does.  Records which thread loaded what."""

    def __init__(self):
        self.calls = []
        self.gate = threading.Event()
        self.gate.set()
        self.entered = threading.Event()
        self.fail = set()

    def __call__(self, path, delta_id, tp_rank, tp_size, prefetch_thread_event=None,
                 discard_prefetching_event=None):
        self.calls.append((delta_id, threading.current_thread().name))
        self.entered.set()
        if discard_prefetching_event is not None and discard_prefetching_event.is_set():
            return None
        if prefetch_thread_event is not None:
            prefetch_thread_event.wait()
            # only background loads stop at the gate: the serving thread is never held
            while not self.gate.wait(0.005):
                if discard_prefetching_event is not None and discard_prefetching_event.is_set():
                    return None
        if discard_prefetching_event is not None and discard_prefetching_event.is_set():
            return None
        if delta_id in self.fail or not os.path.isdir(path):
            raise FileNotFoundError(path)
        return FakeDelta(delta_id)


def req(i, path="/"):
    return DeltaRequest(f"delta-{i}", i, path)


def wait_for(cond, timeout=5.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if cond():
            return True
        time.sleep(0.005)
    return False


def test_delta_request_identity():
    with pytest.raises(ValueError):
        DeltaRequest("base", 0, "/")
    assert req(3) == DeltaRequest("other name", 3, "/elsewhere") and len({req(3), req(3)}) == 1


def test_plain_and_lru_managers_load_failures_and_slot_exhaustion():
    mgr, loader = FakeSlotManager(capacity=2, delta_slots=2), ScriptedLoader()
    w = LRUCacheWorkerDeltaManager(mgr, loader=loader)
    w.set_active_deltas([req(1), req(2)], "mapping-a")
    assert mgr.active == [1, 2] and mgr.mapping == "mapping-a"
    with pytest.raises(RuntimeError, match="delta slots"):        # three deltas, two GPU slots
        w.set_active_deltas([req(1), req(2), req(3)], "mapping-b")
    w.set_active_deltas([req(3)], "mapping-c")                    # host cache full: oldest leaves
    assert set(mgr.registered) == {2, 3}
    with pytest.raises(ValueError, match="load failed"):          # a missing directory
        w.add_delta(req(9, "/definitely/not/here"))
    assert 9 not in mgr.registered
    assert "disk_to_host_s" in w.load_times[3]
    plain = WorkerDeltaManager(FakeSlotManager(), loader=loader)
    plain.set_active_deltas([req(1)], "m")
    plain.set_active_deltas([req(2)], "m")                        # the plain manager drops what left the batch
    assert plain.list_deltas() == {2}


def test_background_prefetch_registers_ahead_of_the_request():
    mgr, loader = FakeSlotManager(), ScriptedLoader()
    w = OverlapLRUCacheWorkerDeltaManager(mgr, loader=loader)
    try:
        w.prefetch_delta(req(5))
        w.prefetch_delta(req(5))                                  # queued once
        assert wait_for(lambda: 5 in mgr.registered)
        assert wait_for(lambda: not w.prefetching_jobqueue)
        assert [c for c in loader.calls if c[0] == 5] == [(5, "delta-prefetch")]
        w.add_delta(req(5))                                       # already on the host: no second load
        assert len([c for c in loader.calls if c[0] == 5]) == 1 and mgr.active == [5]
        # a prefetch that fails is dropped from the queue without disturbing anything
        loader.fail.add(6)
        w.prefetch_delta(req(6))
        assert wait_for(lambda: not w.prefetching_jobqueue)
        assert 6 not in mgr.registered
    finally:
        w.close()
    assert not w._thread.is_alive()


def test_serving_thread_pauses_and_discards_the_background_load():
    mgr, loader = FakeSlotManager(), ScriptedLoader()
    w = OverlapLRUCacheWorkerDeltaManager(mgr, loader=loader)
    try:
        loader.gate.clear()                                       # hold the background load of 7
        w.prefetch_delta(req(7))
        assert wait_for(lambda: w.current_prefetching_request == req(7))
        # the serving thread now needs 7 itself: it aborts the background load and loads at once
        w.add_delta(req(7))
        assert mgr.active == [7] and 7 in mgr.registered
        main_loads = [c for c in loader.calls if c[0] == 7 and c[1] != "delta-prefetch"]
        assert len(main_loads) == 1
        assert 7 not in w.prefetched                              # the background copy was discarded
        assert w.prefetching_thread_event.is_set() and not w.discard_prefetching_event.is_set()
        assert wait_for(lambda: w.current_prefetching_request is None)
        # a different delta in flight is paused, not discarded, while the serving thread loads
        w.prefetch_delta(req(8))
        assert wait_for(lambda: w.current_prefetching_request == req(8))
        w.add_delta(req(9))
        assert 9 in mgr.registered and 8 not in mgr.registered
        loader.gate.set()
        assert wait_for(lambda: 8 in mgr.registered) and 8 in w.prefetched
    finally:
        loader.gate.set()
        w.close()


def test_background_thread_respects_the_host_cache_capacity():
    mgr, loader = FakeSlotManager(capacity=1), ScriptedLoader()
    w = OverlapLRUCacheWorkerDeltaManager(mgr, loader=loader)
    try:
        w.add_delta(req(1))
        w.prefetch_delta(req(2))
        time.sleep(0.1)
        assert 2 not in mgr.registered and [c[0] for c in loader.calls] == [1]   # no room: not loaded
        w.add_delta(req(2))                                       # the serving thread evicts and loads
        assert set(mgr.registered) == {2}
    finally:
        w.close()
