"""Batch loader with the interface of the reference's DataLoader (include/origin/data/dataloader.h,
src/data/dataloader.cpp:11-146):

    loader = DataLoader(inputs, labels, batch_size, shuffle=True)
    while loader.has_next():
        x, t = loader.next()          # x [b, features] float32, t [b] int64, both on the device
    loader.reset()                    # new epoch: indices 0..N-1, reshuffled when shuffle is on

Semantics kept: samples are flattened to `features` values; batches follow the index list in order; the last batch of
an epoch is short unless `drop_last`; next() past the end raises; integer labels come out as int64.  The reference
seeds its shuffle from std::random_device (dataloader.cpp:29-31), so its order is not reproducible; here `seed` makes
it so (None = from the OS, like the reference): epoch e uses the e-th permutation drawn from that generator, in
either mode.  For data-parallel training `shard=(rank, world)` gives every rank the positions rank, rank + world, ... of
the epoch's (common) permutation.

What differs is where the work happens.  The reference assembles each batch on the host one sample at a time and the
training loop copies it to the device.  Here there are two modes:

* resident (default when the data set fits `resident_limit_bytes`): inputs and labels are uploaded ONCE and stay in
  HBM (180 GB per B200 holds every data set of the reference's examples many times over); a batch is one row-gather
  kernel (odl_gather_rows) driven by the shuffled indices, which are uploaded once per epoch.
* staged: the data set stays in host memory; a worker thread gathers the following batches -- across epoch boundaries
  -- into pinned staging buffers (`depth` of them) and copies them with cudaMemcpyAsync on a copy stream while the
  current batch trains; the compute stream waits on the copy's event, the worker on the event of the step that last
  read the buffer.  Without shuffling, batches are contiguous row ranges and are copied straight from the
  (page-locked) data set.
"""
from __future__ import annotations

import queue
import threading

import numpy as np
import torch

from . import capi, dp


class DataLoader:
    def __init__(self, inputs, labels, batch_size: int, shuffle: bool = True, seed: int | None = None,
                 drop_last: bool = False, resident: bool | None = None, resident_limit_bytes: int = 64 << 30,
                 depth: int = 3, pin_limit_bytes: int = 16 << 30, device: int = 0, shard: tuple[int, int] | None = None):
        inputs = np.asarray(inputs, np.float32)
        self.n = int(inputs.shape[0])
        if self.n == 0 or batch_size <= 0:
            raise ValueError("DataLoader: empty data set or non-positive batch size")
        self.host_x = np.ascontiguousarray(inputs.reshape(self.n, -1))
        labels = np.asarray(labels)
        if labels.shape[0] != self.n:
            raise ValueError(f"DataLoader: {self.n} inputs but {labels.shape[0]} labels")
        self.host_t = np.ascontiguousarray(labels.reshape(self.n).astype(np.int64))
        self.features = int(self.host_x.shape[1])
        self.batch_size, self.shuffle, self.drop_last = int(batch_size), bool(shuffle), bool(drop_last)
        self._rng = np.random.default_rng(seed)
        # data parallel: shard = (rank, world); every rank must pass the same seed so that all draw the same permutation
        self.shard = shard
        if shard is not None and (seed is None and shuffle):
            raise ValueError("DataLoader: a sharded, shuffled loader needs an explicit seed shared by all ranks")
        self._orders, self._orders_lock, self._drawn = {}, threading.Lock(), 0
        capi.init(device)
        self.resident = (self.host_x.nbytes <= resident_limit_bytes) if resident is None else bool(resident)
        self.h2d_bytes = 0  # bytes copied host -> device so far (a benchmark reports them per step)
        self.epoch, self.current = 0, 0
        self.indices = self._order_of(0)
        if self.resident:
            self._dev_x = torch.from_numpy(self.host_x).cuda()
            self._dev_t = torch.from_numpy(self.host_t).cuda()
            self.h2d_bytes += self.host_x.nbytes + self.host_t.nbytes
            self._upload_indices()
        else:
            self._device = device
            self._copy_stream = torch.cuda.Stream()
            self._slots = [self._Slot(self.batch_size, self.features) for _ in range(max(2, depth))]
            self._worker, self._pending_release = None, None
            self._pinned_x = None
            if not self.shuffle and self.shard is None and self.host_x.nbytes <= pin_limit_bytes:
                # sequential batches are contiguous row ranges: page-lock the data set itself and copy from it directly
                self._pinned_x = torch.from_numpy(self.host_x).pin_memory()
                self._pinned_t = torch.from_numpy(self.host_t).pin_memory()
            self._start_worker()

    class _Slot:
        def __init__(self, batch, features):
            self.pin_x = torch.empty(batch, features, dtype=torch.float32).pin_memory()
            self.pin_t = torch.empty(batch, dtype=torch.int64).pin_memory()
            self.dev_x = torch.empty(batch, features, dtype=torch.float32, device="cuda")
            self.dev_t = torch.empty(batch, dtype=torch.int64, device="cuda")
            self.ready = torch.cuda.Event()     # the copy into dev_x / dev_t has finished
            self.consumed = torch.cuda.Event()  # the kernels that read dev_x / dev_t have finished
            self.used = False

    # ---- index bookkeeping: DataLoader::reset_indices / has_next / next (dataloader.cpp:17-36, 141-146)
    def _order_of(self, epoch: int) -> np.ndarray:
        """Index list of an epoch; permutations are drawn from the generator strictly in epoch order."""
        with self._orders_lock:
            while self._drawn <= epoch:
                order = np.arange(self.n, dtype=np.int64)
                if self.shuffle:
                    self._rng.shuffle(order)
                if self.shard is not None:
                    order = np.ascontiguousarray(dp.shard_epoch_order(order, *self.shard))
                self._orders[self._drawn] = order
                self._drawn += 1
            for old in [e for e in self._orders if e < epoch - 1]:
                del self._orders[old]
            return self._orders[epoch]

    def _upload_indices(self) -> None:
        self._dev_idx = torch.from_numpy(self.indices).cuda()
        self.h2d_bytes += self.indices.nbytes

    def _rows_at(self, cursor: int) -> int:
        rows = min(self.batch_size, len(self.indices) - cursor)
        return 0 if rows <= 0 or (self.drop_last and rows < self.batch_size) else rows

    def has_next(self) -> bool:
        return self._rows_at(self.current) > 0

    def __len__(self) -> int:
        n = len(self.indices)
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)

    def __iter__(self):
        if self.current:
            self.reset()
        while self.has_next():
            yield self.next()

    def reset(self) -> None:
        """Start the next epoch (a new permutation when shuffling).  At an epoch boundary the staged mode carries on
        without a pause: the worker has already begun staging the next epoch's first batches."""
        finished = not self.has_next()
        if not self.resident and not finished:
            self._stop_worker()  # batches of the abandoned epoch are staged or in flight: drop them
        self.epoch += 1
        self.current = 0
        self.indices = self._order_of(self.epoch)
        if self.resident:
            self._upload_indices()
        elif not finished:
            self._start_worker()

    # ---- staged mode: a worker thread fills pinned buffers and starts their copies ahead of the training loop
    def _start_worker(self) -> None:
        self._free, self._ready, self._stop = queue.Queue(), queue.Queue(), False
        for slot in self._slots:
            self._free.put(slot)
        self._worker = threading.Thread(target=self._stage_forever, args=(self.epoch,), daemon=True)
        self._worker.start()

    def _stop_worker(self) -> None:
        if self._worker is None:
            return
        self._stop = True
        self._free.put(None)
        self._worker.join()
        self._worker, self._pending_release = None, None
        torch.cuda.synchronize()  # nothing still reads or writes the slots

    def _stage_forever(self, epoch: int) -> None:
        torch.cuda.set_device(self._device)
        try:
            while not self._stop:
                indices, cursor = self._order_of(epoch), 0
                while True:
                    rows = self._rows_at(cursor)
                    if rows == 0:
                        break
                    slot = self._free.get()
                    if slot is None or self._stop:
                        return
                    if slot.used:
                        slot.consumed.synchronize()
                    if self._pinned_x is not None:
                        src_x, src_t = self._pinned_x[cursor:cursor + rows], self._pinned_t[cursor:cursor + rows]
                    else:
                        ids = indices[cursor:cursor + rows]
                        np.take(self.host_x, ids, axis=0, out=slot.pin_x.numpy()[:rows])
                        np.take(self.host_t, ids, out=slot.pin_t.numpy()[:rows])
                        src_x, src_t = slot.pin_x[:rows], slot.pin_t[:rows]
                    with torch.cuda.stream(self._copy_stream):
                        slot.dev_x[:rows].copy_(src_x, non_blocking=True)
                        slot.dev_t[:rows].copy_(src_t, non_blocking=True)
                        slot.ready.record(self._copy_stream)
                    self.h2d_bytes += rows * (self.features * 4 + 8)
                    self._ready.put((epoch, slot, rows))
                    cursor += rows
                epoch += 1
        except BaseException as e:  # surface the failure in next() instead of leaving it waiting
            self._ready.put(e)

    def next(self):
        rows = self._rows_at(self.current)
        if rows == 0:
            raise RuntimeError("DataLoader::next() called when no more data available. Use has_next() to check before "
                               "calling next().")
        if self.resident:
            x = torch.empty(rows, self.features, dtype=torch.float32, device="cuda")
            t = torch.empty(rows, dtype=torch.int64, device="cuda")
            capi.call("odl_gather_rows", self._dev_x.data_ptr(), self.features, self.n,
                      self._dev_idx.data_ptr() + 8 * self.current, rows, self.features, x.data_ptr(), self.features,
                      self._dev_t.data_ptr(), t.data_ptr(), capi.stream_handle())
            self.current += rows
            return x, t
        self.release()
        item = self._ready.get(timeout=600)
        if isinstance(item, BaseException):
            raise item
        epoch, slot, got = item
        assert epoch == self.epoch and got == rows, (epoch, self.epoch, got, rows)
        torch.cuda.current_stream().wait_event(slot.ready)
        self.current += rows
        self._pending_release = slot
        return slot.dev_x[:rows], slot.dev_t[:rows]

    def release(self) -> None:
        """Staged mode: the kernels that read the last batch have been enqueued on the current stream, so its buffers
        may be refilled once they finish.  The loader calls this itself at the next next(); calling it right after the
        training step lets the worker start refilling one step earlier."""
        if self.resident:
            return
        slot, self._pending_release = self._pending_release, None
        if slot is not None:
            slot.consumed.record(torch.cuda.current_stream())
            slot.used = True
            self._free.put(slot)

    def close(self) -> None:
        if not self.resident:
            self._stop_worker()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
