"""Host-side admission logic of the decode engine, without a GPU: the engine object is built
around a fake slot manager and a real (CPU) block free list, so only the decisions are tested --
which sequences join, which delta is evicted, which swap-ins are started and when a sequence
whose delta is still in flight may join (the role of the reference's scheduler limits,
serving/vllm/core/scheduler.py:359-366,528-535)."""
from collections import OrderedDict

import torch

from deltazip_b200.engine import DecodeEngine, Sequence
from deltazip_b200.llama import PagedKVCache


class FakeManager:
    def __init__(self, slots, known):
        self.delta_slots = slots
        self.known = set(known)
        self._active_deltas = OrderedDict()
        self._loading = {}
        self.log = []

    def get_delta(self, d):
        return object() if d in self.known else None

    def activate_delta(self, d):
        self._loading.pop(d, None)
        self._active_deltas[d] = None
        self.log.append(("activate", d))
        return True

    def deactivate_delta(self, d):
        self._active_deltas.pop(d)
        self.log.append(("evict", d))
        return True

    def prefetch_delta(self, d):
        self._loading[d] = len(self._loading)
        self.log.append(("prefetch", d))


def make_engine(slots, known, max_seqs=8, kv_blocks=64, block_size=16):
    eng = DecodeEngine.__new__(DecodeEngine)            # no model, no device
    eng.block_size, eng.max_seqs = block_size, max_seqs
    eng.manager = FakeManager(slots, known)
    eng.cache = PagedKVCache(0, kv_blocks, 1, block_size, torch.float16, "cpu")
    eng.running, eng._dirty, eng.swap_ins = [], False, 0
    return eng


def seq(i, d, length=100, new=28):
    return Sequence(seq_id=i, delta_id=d, length=length, max_new=new)


def test_admit_takes_sequences_while_slots_blocks_and_batch_allow():
    eng = make_engine(slots=2, known={1, 2, 3})
    waiting = [seq(0, 1), seq(1, 2), seq(2, 3), seq(3, 1), seq(4, 0), seq(5, 9)]
    got = eng.admit(waiting)
    # deltas 1 and 2 fill the two slots; 3 finds both in use; 9 is unknown; the base model needs none
    assert [s.seq_id for s in got] == [0, 1, 3, 4]
    assert [s.seq_id for s in waiting] == [2, 5]
    assert eng.manager.log == [("activate", 1), ("activate", 2)]
    assert all(len(s.blocks) == 8 for s in got) and len(eng.cache.free) == 64 - 32
    # once the sequences of delta 1 are gone, delta 3 may evict it (least recently used, unused)
    for s in [x for x in eng.running if x.delta_id == 1]:
        eng.retire(s)
    got = eng.admit(waiting)
    assert [s.seq_id for s in got] == [2] and ("evict", 1) in eng.manager.log
    assert list(eng.manager._active_deltas) == [2, 3]


def test_admit_respects_batch_size_and_kv_blocks():
    eng = make_engine(slots=4, known={1}, max_seqs=2)
    waiting = [seq(i, 1) for i in range(4)]
    assert len(eng.admit(waiting)) == 2 and len(waiting) == 2
    eng = make_engine(slots=4, known={1}, kv_blocks=10)
    waiting = [seq(0, 1), seq(1, 1, length=10, new=6), seq(2, 1)]
    got = eng.admit(waiting)                                 # 8 blocks, then 1 block, then none left
    assert [s.seq_id for s in got] == [0, 1] and len(eng.cache.free) == 1


def test_overlapped_admission_starts_the_swap_in_and_admits_when_it_has_landed():
    eng = make_engine(slots=1, known={1, 2})
    landed = set()
    waiting = [seq(0, 1), seq(1, 1), seq(2, 2)]
    assert eng.admit_overlapped(waiting, ready=lambda d: d in landed) == []
    assert eng.manager.log == [("prefetch", 1)] and eng.swap_ins == 1      # one upload for both
    assert eng.admit_overlapped(waiting, ready=lambda d: d in landed) == []   # still in flight
    landed.add(1)
    got = eng.admit_overlapped(waiting, ready=lambda d: d in landed)
    assert [s.seq_id for s in got] == [0, 1] and ("activate", 1) in eng.manager.log
    # delta 2 has to wait for the only slot: nothing is evicted under running sequences
    assert [s.seq_id for s in waiting] == [2] and ("evict", 1) not in eng.manager.log
    for s in list(eng.running):
        eng.retire(s)
    assert eng.admit_overlapped(waiting, ready=lambda d: d in landed) == []
    assert eng.manager.log[-2:] == [("evict", 1), ("prefetch", 2)] and eng.swap_ins == 2
