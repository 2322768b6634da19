"""Per-worker delta management: loading deltas from disk into the pinned host cache, on the
caller's thread or ahead of time on a background thread, and putting them on the GPU.

Counterpart of serving/vllm/delta/worker_manager.py: `WorkerDeltaManager` :62-187,
`LRUCacheWorkerDeltaManager` :190-246 and `OverlapLRUCacheWorkerDeltaManager` :248-376 with its
background loader (`_load_delta_background` :256-289), `prefetch_delta` :324-333 and the two
threading events that let the serving thread pause the loader (`prefetching_thread_event`) or
make it abandon the delta it is loading (`discard_prefetching_event`) :335-364, and
`DeltaRequest` (serving/vllm/delta/request.py:4-25).

Differences by design: the background thread can be stopped (`close`), the job queue is guarded
by a lock, the loader is injectable (tests drive the thread logic with a fake loader and a fake
slot manager, no GPU), and what a load cost is kept per delta (`load_times`) next to the
per-request `cpu_loading_time` / `gpu_loading_time` stamps.
"""
from __future__ import annotations

import logging
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Set

logger = logging.getLogger(__name__)

CHECK_QUEUE_INTERVAL = 0.01


@dataclass
class DeltaRequest:
    """A delta the engine wants served: a name, a positive integer id and a local directory."""
    delta_name: str
    delta_int_id: int
    delta_local_path: str

    def __post_init__(self):
        if self.delta_int_id < 1:
            raise ValueError(f"delta ids start at 1 (0 is the base model), got {self.delta_int_id}")

    @property
    def delta_id(self) -> int:
        return self.delta_int_id

    def __eq__(self, other) -> bool:
        return isinstance(other, DeltaRequest) and self.delta_int_id == other.delta_int_id

    def __hash__(self) -> int:
        return self.delta_int_id


def _default_loader(path: str, delta_id: int, tp_rank: int, tp_size: int,
                    prefetch_thread_event=None, discard_prefetching_event=None):
    from .models import DeltaModel
    return DeltaModel.from_checkpoint(path, delta_id, tp_rank=tp_rank, tp_size=tp_size,
                                      prefetch_thread_event=prefetch_thread_event,
                                      discard_prefetching_event=discard_prefetching_event)


class WorkerDeltaManager:
    """Loads deltas when they are first requested and keeps them registered; the number of
    distinct deltas of a batch may not exceed the GPU slots."""

    def __init__(self, delta_manager, tp_rank: int = 0, tp_size: int = 1,
                 loader: Optional[Callable] = None):
        self._delta_manager = delta_manager
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self._loader = loader or _default_loader
        self.load_times: Dict[int, Dict[str, float]] = {}

    # -- loading -------------------------------------------------------------------
    def _load_delta(self, delta_request: DeltaRequest, prefetch_event=None, discard_event=None):
        """Disk -> host.  Any failure (missing directory, truncated file, tensors that do not
        describe a servable delta) is logged and turned into None, as the reference does
        (worker_manager.py:143-158); the caller decides what a missing delta means."""
        t0 = time.perf_counter()
        try:
            delta = self._loader(delta_request.delta_local_path, delta_request.delta_int_id,
                                 self.tp_rank, self.tp_size, prefetch_thread_event=prefetch_event,
                                 discard_prefetching_event=discard_event)
        except Exception as exc:                                   # noqa: BLE001 (see docstring)
            logger.error("loading delta %s from %s failed: %s", delta_request.delta_int_id,
                         delta_request.delta_local_path, exc)
            return None
        if delta is not None:
            self.load_times.setdefault(delta_request.delta_int_id, {})["disk_to_host_s"] = \
                time.perf_counter() - t0
        return delta

    def _activate_delta(self, delta_request: DeltaRequest) -> None:
        t0 = time.perf_counter()
        self._delta_manager.activate_delta(delta_request.delta_int_id)
        self.load_times.setdefault(delta_request.delta_int_id, {})["activate_call_s"] = \
            time.perf_counter() - t0

    # -- the runner's entry points ---------------------------------------------------
    def set_active_deltas(self, delta_requests: List[DeltaRequest], delta_mapping,
                          sequence_groups: Optional[list] = None) -> None:
        self._apply_deltas(delta_requests, sequence_groups or [])
        self._delta_manager.set_delta_mapping(delta_mapping)

    def _apply_deltas(self, delta_requests: List[DeltaRequest], sequence_groups: list) -> None:
        wanted = {r.delta_int_id: r for r in delta_requests}
        if len(wanted) > self._delta_manager.delta_slots:
            raise RuntimeError(f"the batch names {len(wanted)} deltas, the GPU has "
                               f"{self._delta_manager.delta_slots} delta slots")
        have = self.list_deltas()
        for delta_id in have - set(wanted):
            self.remove_delta(delta_id)
        for delta_id in set(wanted) - have:
            self.add_delta(wanted[delta_id], sequence_groups)

    def add_delta(self, delta_request: DeltaRequest, sequence_groups: Optional[list] = None) -> bool:
        if delta_request.delta_int_id in self.list_deltas():
            return False
        delta = self._load_delta(delta_request)
        _stamp(sequence_groups, "maybe_set_cpu_loading_time")
        loaded = self._delta_manager.add_delta(delta)
        self._delta_manager.activate_delta(delta.id)
        _stamp(sequence_groups, "maybe_set_gpu_loading_time")
        return loaded

    def remove_delta(self, delta_id: int) -> bool:
        return self._delta_manager.remove_delta(delta_id)

    def remove_all_deltas(self):
        return self._delta_manager.remove_all_deltas()

    def list_deltas(self) -> Set[int]:
        return set(self._delta_manager.list_deltas())

    def close(self) -> None:
        pass


def _stamp(sequence_groups, method: str) -> None:
    for sg in sequence_groups or []:
        fn = getattr(sg, method, None)
        if fn is not None:
            fn(time.time())


class LRUCacheWorkerDeltaManager(WorkerDeltaManager):
    """Keeps deltas registered across batches; the least recently used one leaves the host cache
    when a new one needs room (worker_manager.py:190-246)."""

    def _apply_deltas(self, delta_requests: List[DeltaRequest], sequence_groups: list) -> None:
        wanted = {r.delta_int_id: r for r in delta_requests}
        if len(wanted) > self._delta_manager.delta_slots:
            raise RuntimeError(f"the batch names {len(wanted)} deltas, the GPU has "
                               f"{self._delta_manager.delta_slots} delta slots")
        for request in wanted.values():
            self.add_delta(request, sequence_groups)

    def add_delta(self, delta_request: DeltaRequest, sequence_groups: Optional[list] = None) -> bool:
        if delta_request.delta_int_id not in self.list_deltas():
            if len(self._delta_manager) + 1 > self._delta_manager.capacity:
                self._delta_manager.remove_oldest_delta()
            delta = self._load_delta(delta_request)
            loaded = self._delta_manager.add_delta(delta)
        else:
            loaded = self._delta_manager.get_delta(delta_request.delta_int_id) is not None
        _stamp(sequence_groups, "maybe_set_cpu_loading_time")
        self._activate_delta(delta_request)
        _stamp(sequence_groups, "maybe_set_gpu_loading_time")
        return loaded


class OverlapLRUCacheWorkerDeltaManager(LRUCacheWorkerDeltaManager):
    """LRU manager with a background thread that loads queued deltas from disk into the host
    cache while the GPU decodes (worker_manager.py:248-376).

    `prefetching_thread_event` set = the loader may run; the serving thread clears it while it
    loads a delta itself (it has priority) and sets it again afterwards.
    `discard_prefetching_event` set = the loader abandons the delta it is loading (the serving
    thread is loading the same one)."""

    def __init__(self, delta_manager, tp_rank: int = 0, tp_size: int = 1,
                 loader: Optional[Callable] = None, start: bool = True):
        super().__init__(delta_manager, tp_rank, tp_size, loader)
        self.prefetching_thread_event = threading.Event()
        self.discard_prefetching_event = threading.Event()
        self.prefetching_jobqueue: List[DeltaRequest] = []
        self.current_prefetching_request: Optional[DeltaRequest] = None
        self._queue_lock = threading.Lock()
        self._manager_lock = threading.RLock()       # registry updates from both threads
        self._stop = threading.Event()
        self.prefetched: List[int] = []               # ids the background thread registered
        self.prefetching_thread_event.set()
        self._thread = threading.Thread(target=self._load_delta_background, daemon=True,
                                        name="delta-prefetch")
        if start:
            self._thread.start()

    # -- background thread -------------------------------------------------------------
    def _load_delta_background(self) -> None:
        while not self._stop.is_set():
            with self._queue_lock:
                jobs = list(self.prefetching_jobqueue)
            for request in jobs:
                if self._stop.is_set():
                    return
                if request.delta_int_id not in self.list_deltas():
                    with self._manager_lock:
                        full = len(self._delta_manager) + 1 > self._delta_manager.capacity
                    if full:
                        break                                    # no room: try again later
                    # wait (in short slices, so that close() is honoured) until allowed to run
                    while not self.prefetching_thread_event.wait(0.05):
                        if self._stop.is_set():
                            return
                    self.current_prefetching_request = request
                    delta = self._load_delta(request, prefetch_event=self.prefetching_thread_event,
                                             discard_event=self.discard_prefetching_event)
                    if delta is not None and not self.discard_prefetching_event.is_set():
                        with self._manager_lock:
                            if request.delta_int_id not in self.list_deltas():
                                self._delta_manager.add_delta(delta)
                                self.prefetched.append(request.delta_int_id)
                    self.current_prefetching_request = None
                with self._queue_lock:
                    if request in self.prefetching_jobqueue:
                        self.prefetching_jobqueue.remove(request)
            self._stop.wait(CHECK_QUEUE_INTERVAL)

    def prefetch_delta(self, delta_request: DeltaRequest) -> None:
        """Queues a delta for the background loader (no-op when it is registered or queued)."""
        with self._queue_lock:
            if delta_request.delta_int_id not in self.list_deltas() and \
                    delta_request not in self.prefetching_jobqueue:
                self.prefetching_jobqueue.append(delta_request)

    # -- serving thread ------------------------------------------------------------------
    def add_delta(self, delta_request: DeltaRequest, sequence_groups: Optional[list] = None) -> bool:
        if delta_request.delta_int_id not in self.list_deltas():
            # missed prefetch: load on this thread, which has priority over the loader
            self.prefetching_thread_event.clear()
            try:
                current = self.current_prefetching_request
                if current is not None and current.delta_int_id == delta_request.delta_int_id:
                    self.discard_prefetching_event.set()
                with self._queue_lock:
                    if delta_request in self.prefetching_jobqueue:
                        self.prefetching_jobqueue.remove(delta_request)
                delta = self._load_delta(delta_request)
                with self._manager_lock:
                    if delta_request.delta_int_id not in self.list_deltas():
                        if len(self._delta_manager) + 1 > self._delta_manager.capacity:
                            self._delta_manager.remove_oldest_delta()
                        loaded = self._delta_manager.add_delta(delta)
                    else:
                        loaded = True
            finally:
                self.prefetching_thread_event.set()
                if self.discard_prefetching_event.is_set():
                    # let the loader notice the flag before it is lowered again
                    deadline = time.time() + 1.0
                    while self.current_prefetching_request is not None and time.time() < deadline:
                        time.sleep(0.001)
                    self.discard_prefetching_event.clear()
        else:
            loaded = self._delta_manager.get_delta(delta_request.delta_int_id) is not None
        _stamp(sequence_groups, "maybe_set_cpu_loading_time")
        with self._manager_lock:
            self._activate_delta(delta_request)
        _stamp(sequence_groups, "maybe_set_gpu_loading_time")
        return loaded

    def close(self) -> None:
        """Stops the background thread (it finishes the file it is reading)."""
        self._stop.set()
        self.prefetching_thread_event.set()
        if self._thread.is_alive():
            self._thread.join(timeout=10)
