"""Pipelined loading: batch k+1 of files is read while the caller consumes the tensors of
batch k.

Same classes, arguments and iteration contract as upstream ``fastsafetensors/parallel_loader.py``
(``PipelineParallel``, ``ParallelLoader``, ``iterate_weights`` yielding ``(key, tensor)`` in
``key_to_rank_lidx`` order, batches of ``world_size`` files with file ``i`` of a batch owned by
rank ``i``; ``queue_size`` -1 / 0 / N as upstream defines them).  Two things differ.

* Where the overlap lives.  Upstream runs ``copy_files_to_device`` of the next batch on a Python
  producer thread and hands batches over through a queue (``parallel_loader.py:284-308``).  Here
  the native reader is the producer: the reads of the batches ahead are *queued* with
  ``copy_files_to_device(wait=False)`` (double- or N-buffered file images, filled by the reader's
  worker threads through its pinned ring) and each file is waited for when its first tensor is
  taken.  No Python thread, no hand-over between threads.  ``producer_thread=True`` (or
  ``FST_B200_PIPELINE_THREAD=1``) selects upstream's arrangement instead.
* With more than one rank upstream broadcasts every tensor on its own
  (``parallel_loader.py:337-350`` -> ``tensor_factory.py:128-143``, a collective and a device
  synchronisation per tensor); here each FILE image is broadcast once
  (``FilesBufferOnDevice.replicate_all``) and the tensors are views of the received images, so a
  batch costs ``world_size`` collectives instead of one per tensor.
"""

from __future__ import annotations

import os
import queue
import threading
import time
from typing import Any, Generator, List, Optional, Tuple, Union

try:
    from tqdm.auto import tqdm

    _TQDM_AVAILABLE = True
except ImportError:  # pragma: no cover
    _TQDM_AVAILABLE = False

    def tqdm(iterable, *args, **kwargs):
        return iterable

from . import cpp as fstcpp
from .common import SingleGroup
from .loader import BaseSafeTensorsFileLoader, SafeTensorsFileLoader

_BAR_FORMAT = "{desc}: {percentage:3.0f}% Completed | {n_fmt}/{total_fmt} [{elapsed}<{remaining}, {rate_fmt}]\n"


def enable_tqdm(use_tqdm_on_load: bool, framework=None) -> bool:
    """Progress bar on global rank 0 only (and only if tqdm is installed)."""
    rank = framework.get_global_rank() if framework is not None else 0
    return _TQDM_AVAILABLE and use_tqdm_on_load and rank == 0


class TimingContext:
    """``with TimingContext("step", log):`` measures a block in milliseconds."""

    def __init__(self, name: str, logger=None, batch_id=None, threshold_ms: float = 0,
                 log_on_exit: bool = True):
        self.name, self.logger, self.batch_id = name, logger, batch_id
        self.threshold_ms, self.log_on_exit = threshold_ms, log_on_exit
        self.start_time: Optional[float] = None
        self.elapsed_ms = 0.0

    def __enter__(self):
        self.start_time = time.time()
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.elapsed_ms = (time.time() - self.start_time) * 1000
        if self.logger and self.log_on_exit and (self.elapsed_ms >= self.threshold_ms or exc_type):
            prefix = f"Batch {self.batch_id}: " if self.batch_id is not None else ""
            self.logger(f"{prefix}{self.name} took {self.elapsed_ms:.3f} ms")
        return False


class FileBatch:
    """One batch of files resident in device memory, with its load timings."""

    def __init__(self, fb, keys: List[str], batch_id: int):
        self.fb = fb
        self.keys = keys
        self.batch_id = batch_id
        self.add_filenames_time: Optional[float] = None
        self.copy_files_time: Optional[float] = None
        self.load_time: Optional[float] = None


class PipelineParallel:
    """Producer/consumer pipeline over batches of ``world_size`` files.

    ``queue_size``: ``N > 0`` up to N loaded batches wait in the queue; ``0`` the producer starts
    the next batch as soon as the consumer has taken the previous one; ``-1`` only after the
    consumer has finished (closed) the previous one.  Device memory in flight is about
    ``(1 + max(queue_size, 0) + 1)`` batches.
    """

    def __init__(self, pg: Optional[Any], loader: BaseSafeTensorsFileLoader, hf_weights_files: List[str],
                 max_concurrent_producers: int = 1, queue_size: int = 0, use_tqdm_on_load: bool = True,
                 producer_thread: Optional[bool] = None, **kwargs):
        if max_concurrent_producers != 1:
            raise ValueError(
                f"max_concurrent_producers must be 1 (got {max_concurrent_producers}). "
                "Concurrent producers > 1 are not yet supported because broadcast "
                "batches must be processed in strict order across all ranks."
            )
        self.loader = loader
        # the group as the caller passed it (None = single process), as upstream sizes its batches
        # (parallel_loader.py:150-159); anything with size() and rank() will do
        self.pg = pg if pg is not None else SingleGroup()
        self.hf_weights_files = hf_weights_files
        self.max_concurrent_producers = max_concurrent_producers
        self.queue_size = queue_size
        self.use_tqdm_on_load = use_tqdm_on_load
        world = self.pg.size()
        self.weight_files_batches = [hf_weights_files[i:i + world]
                                     for i in range(0, len(hf_weights_files), world)]
        self.batch_queue: "queue.Queue[Union[FileBatch, Exception, None]]" = queue.Queue(
            maxsize=max(1, queue_size))
        self.stop_event = threading.Event()
        self.error_event = threading.Event()
        self.error_info: Optional[str] = None
        # modes 0 and -1: one ticket; the producer takes it before copying a batch and the consumer
        # gives it back when it has taken (0) or finished (-1) that batch
        self._ticket: Optional[threading.Semaphore] = threading.Semaphore(1) if queue_size <= 0 else None
        self.print_log = os.getenv("FASTSAFETENSORS_DEBUG", "false").lower() == "true"
        self.log_prefix = f"PG{self.pg.rank()}"
        self.need_clone = world == 1
        if producer_thread is None:
            producer_thread = os.getenv("FST_B200_PIPELINE_THREAD", "0") == "1"
        self.producer_thread = bool(producer_thread)
        fstcpp.set_gil_release(True)

    # ------------------------------------------------------------------ logging
    def _log_message(self, message: str, is_error: bool = False) -> None:
        if self.print_log or is_error:
            now = time.time()
            stamp = time.strftime("%Y-%m-%d %H:%M:%S", time.localtime(now)) + f".{int(now % 1 * 1000):03d}"
            print(f"[{self.log_prefix}] {stamp} - {message}", flush=True)

    # ------------------------------------------------------------------ producer
    def _load_batch(self, batch_id: int, files: List[str], wait: bool = True) -> Optional[FileBatch]:
        with TimingContext("add_filenames", self._log_message, batch_id) as t_add:
            self.loader.add_filenames({i: [f] for i, f in enumerate(files)})
        if wait and self._ticket is not None:
            while not self._ticket.acquire(timeout=0.2):
                if self.stop_event.is_set():
                    return None
        with TimingContext("copy_files_to_device", self._log_message, batch_id) as t_copy:
            fb = self.loader.copy_files_to_device() if wait else self.loader.copy_files_to_device(wait=False)
        batch = FileBatch(fb, list(fb.key_to_rank_lidx.keys()), batch_id)
        batch.add_filenames_time, batch.copy_files_time = t_add.elapsed_ms, t_copy.elapsed_ms
        batch.load_time = t_add.elapsed_ms + t_copy.elapsed_ms
        self.loader.reset()
        return batch

    def _put(self, item) -> bool:
        while not self.stop_event.is_set():
            try:
                self.batch_queue.put(item, timeout=0.2)
                return True
            except queue.Full:
                continue
        return False

    def _producer_worker(self) -> None:
        try:
            for batch_id, files in enumerate(self.weight_files_batches):
                if self.stop_event.is_set():
                    return
                batch = self._load_batch(batch_id, files)
                if batch is None:
                    return
                if not self._put(batch):
                    batch.fb.close()   # the consumer went away
                    return
        except Exception as e:  # noqa: BLE001
            self.error_info = f"Producer failed: {e}"
            self.error_event.set()
            self._put(e)
            return
        self._put(None)

    # ------------------------------------------------------------------ consumer
    def _consume_batch(self, batch: FileBatch) -> Generator[Tuple[str, Any], None, None]:
        try:
            with TimingContext("get_tensor", self._log_message, batch.batch_id) as t_get:
                if not self.need_clone:
                    batch.fb.replicate_all()      # one broadcast per file; tensors become views
                for key in batch.keys:
                    tensor = batch.fb.get_tensor(key)
                    if self.need_clone:
                        tensor = tensor.clone()
                    yield key, tensor
        finally:
            with TimingContext("fb.close", self._log_message, batch.batch_id) as t_close:
                batch.fb.close()
            if self.producer_thread and self._ticket is not None and self.queue_size < 0:
                self._ticket.release()
        self._log_message(
            f"Batch {batch.batch_id} summary: add_filenames={batch.add_filenames_time:.3f}ms, "
            f"copy_files={batch.copy_files_time:.3f}ms, get_tensor_total={t_get.elapsed_ms:.3f}ms, "
            f"close={t_close.elapsed_ms:.3f}ms, num_keys={len(batch.keys)}")

    def iterate_weights(self) -> Generator[Tuple[str, Any], None, None]:
        """Yield ``(key, tensor)`` for every tensor of every file, batch by batch."""
        if self.producer_thread:
            yield from self._iterate_with_producer_thread()
        else:
            yield from self._iterate_native()

    def _iterate_native(self) -> Generator[Tuple[str, Any], None, None]:
        """The native reader as producer.  ``ahead`` batches beyond the one being consumed have
        their reads queued: none for ``queue_size`` -1 (the next batch starts when this one is
        closed), one for 0, ``queue_size + 1`` for N > 0 -- the same number of file images in
        device memory as upstream's queue holds.  A failure to queue a batch (a missing file,
        say) is kept and raised when the consumer reaches that batch, as upstream's queue
        delivers the producer's exception in order."""
        ahead = 0 if self.queue_size < 0 else self.queue_size + 1
        batches = self.weight_files_batches
        queued: "List[Union[FileBatch, Exception]]" = []
        next_id = 0
        bar = tqdm(total=len(batches), desc="Loading fastsafetensors checkpoint shards",
                   disable=not enable_tqdm(self.use_tqdm_on_load, self.loader.framework),
                   bar_format=_BAR_FORMAT) if _TQDM_AVAILABLE else None

        def top_up(target: int) -> None:
            nonlocal next_id
            while len(queued) < target and next_id < len(batches):
                if queued and isinstance(queued[-1], Exception):
                    return                     # nothing is queued behind a failed batch
                try:
                    item = self._load_batch(next_id, batches[next_id], wait=False)
                except Exception as e:  # noqa: BLE001
                    self.error_info = f"Producer failed: {e}"
                    self.error_event.set()
                    item = e
                    self.loader.reset()
                queued.append(item)
                next_id += 1

        try:
            top_up(1)
            while queued:
                item = queued.pop(0)
                if isinstance(item, Exception):
                    raise item
                top_up(ahead)                  # reads of the batches ahead run while this one is consumed
                yield from self._consume_batch(item)
                if bar is not None:
                    bar.update(1)
                top_up(1)
        finally:
            self.stop_event.set()
            if bar is not None:
                bar.close()
            for left in queued:               # batches that were queued but never consumed
                if isinstance(left, FileBatch):
                    left.fb.close()

    def _iterate_with_producer_thread(self) -> Generator[Tuple[str, Any], None, None]:
        """Upstream's arrangement: a Python producer thread and a queue of loaded batches."""
        producer = threading.Thread(target=self._producer_worker, name="fst-producer", daemon=True)
        producer.start()
        bar = tqdm(total=len(self.weight_files_batches), desc="Loading fastsafetensors checkpoint shards",
                   disable=not enable_tqdm(self.use_tqdm_on_load, self.loader.framework),
                   bar_format=_BAR_FORMAT) if _TQDM_AVAILABLE else None
        done = 0
        try:
            while done < len(self.weight_files_batches):
                item = self.batch_queue.get()
                if self._ticket is not None and self.queue_size == 0:
                    self._ticket.release()
                if item is None:
                    break
                if isinstance(item, Exception):
                    raise item
                yield from self._consume_batch(item)
                done += 1
                if bar is not None:
                    bar.update(1)
        finally:
            self.stop_event.set()
            producer.join(timeout=5)
            if bar is not None:
                bar.close()
            # batches that were loaded but never consumed
            while True:
                try:
                    left = self.batch_queue.get_nowait()
                except queue.Empty:
                    break
                if isinstance(left, FileBatch):
                    left.fb.close()

    def close(self) -> None:
        self.loader.close()


class ParallelLoader(PipelineParallel):
    """``PipelineParallel`` that builds its own ``SafeTensorsFileLoader``.

    Example::

        it = ParallelLoader(None, files, queue_size=0, device="cuda:0", nogds=True)
        for key, tensor in it.iterate_weights():
            ...
        it.close()
    """

    def __init__(self, pg: Optional[Any], hf_weights_files: List[str], max_concurrent_producers: int = 1,
                 queue_size: int = 0, use_tqdm_on_load: bool = True, device: Any = "cpu",
                 bbuf_size_kb: int = 16 * 1024, max_threads: int = 16, nogds: bool = False,
                 set_numa: bool = True, debug_log: bool = False, framework="pytorch",
                 producer_thread: Optional[bool] = None, **kwargs):
        loader = SafeTensorsFileLoader(pg, device, bbuf_size_kb=bbuf_size_kb, max_threads=max_threads,
                                       nogds=nogds, disable_cache=True, set_numa=set_numa,
                                       debug_log=debug_log, framework=framework, **kwargs)
        super().__init__(pg, loader, hf_weights_files, max_concurrent_producers, queue_size,
                         use_tqdm_on_load, producer_thread=producer_thread)
