"""Host / NVMe offload of tensors with asynchronous copies.

reference: ``src/distributed/zero_sharding.zig:183-247`` (``offloadToCPU`` synchronous D2H,
``offloadToNVMe`` / ``loadFromNVMe`` seek + write / read of one file, ``asyncOffload`` /
``asyncPrefetch`` through a 1 GiB pinned staging buffer on per-GPU streams), ``src/io.zig:5-152``
(``AsyncIO``: queued file reads / writes with pinned buffers), YAML flags ``runtime.cpu_offload``,
``runtime.nvme_offload``, ``runtime.nvme_path``.

``HostOffloader`` keeps a pinned mirror per registered tensor and moves data on a side stream;
``NvmeStore`` persists mirrors to one file per tensor with positional I/O on a worker thread.
With 180 GB per GPU the benchmark configurations never need this; it exists for larger models.
"""
from __future__ import annotations

import os
import queue
import threading
from typing import Dict, Optional

import torch


class HostOffloader:
    def __init__(self, device: torch.device):
        self.device = device
        self.cuda = device.type == "cuda"
        self.stream = torch.cuda.Stream(device) if self.cuda else None
        self.mirrors: Dict[str, torch.Tensor] = {}
        self.events: Dict[str, object] = {}

    def register(self, name: str, t: torch.Tensor) -> None:
        m = torch.empty(t.shape, dtype=t.dtype, device="cpu")
        if self.cuda:
            m = m.pin_memory()
        self.mirrors[name] = m

    def offload(self, name: str, t: torch.Tensor, non_blocking: bool = True) -> None:
        """device → pinned host. The copy runs on the side stream after the producer stream's work."""
        if name not in self.mirrors:
            self.register(name, t)
        if not self.cuda:
            self.mirrors[name].copy_(t)
            return
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            self.mirrors[name].copy_(t, non_blocking=non_blocking)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.events[name] = ev

    def prefetch(self, name: str, out: torch.Tensor) -> None:
        """pinned host → device on the side stream; call :meth:`wait` before using ``out``."""
        if not self.cuda:
            out.copy_(self.mirrors[name])
            return
        with torch.cuda.stream(self.stream):
            out.copy_(self.mirrors[name], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.events[name] = ev

    def wait(self, name: Optional[str] = None) -> None:
        if not self.cuda:
            return
        if name is None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        elif name in self.events:
            torch.cuda.current_stream(self.device).wait_event(self.events[name])

    def synchronize(self) -> None:
        if self.cuda:
            self.stream.synchronize()


class NvmeStore:
    """One file per tensor under ``root``; writes and reads are queued to a worker thread."""

    def __init__(self, root: str):
        self.root = root
        os.makedirs(root, exist_ok=True)
        self._q: "queue.Queue" = queue.Queue()
        self._err: Optional[BaseException] = None
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _path(self, name: str) -> str:
        return os.path.join(self.root, name.replace("/", "_") + ".bin")

    def _run(self) -> None:
        while True:
            job = self._q.get()
            if job is None:
                return
            kind, name, t, done = job
            try:
                buf = t.view(torch.uint8).numpy() if t.dtype != torch.bfloat16 else t.view(torch.int16).numpy().view("uint8")
                if kind == "w":
                    fd = os.open(self._path(name), os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o644)
                    try:
                        os.pwrite(fd, buf.tobytes(), 0)
                    finally:
                        os.close(fd)
                else:
                    fd = os.open(self._path(name), os.O_RDONLY)
                    try:
                        data = os.pread(fd, buf.nbytes, 0)
                    finally:
                        os.close(fd)
                    if len(data) != buf.nbytes:
                        raise IOError(f"short read for {name}")
                    buf.reshape(-1)[:] = memoryview(data)
            except BaseException as e:      # noqa: BLE001 - surfaced by flush()
                self._err = e
            finally:
                done.set()

    def write(self, name: str, host_tensor: torch.Tensor) -> threading.Event:
        done = threading.Event()
        self._q.put(("w", name, host_tensor.contiguous(), done))
        return done

    def read(self, name: str, host_tensor: torch.Tensor) -> threading.Event:
        done = threading.Event()
        self._q.put(("r", name, host_tensor, done))
        return done

    def flush(self) -> None:
        done = threading.Event()
        self._q.put(("w", "__flush__", torch.zeros(1, dtype=torch.uint8), done))
        done.wait()
        if self._err is not None:
            e, self._err = self._err, None
            raise e

    def close(self) -> None:
        self._q.put(None)
        self._t.join()


class OptimizerStateOffload:
    """Keeps the optimizer's moment buffers on the host (and optionally on NVMe) between steps.

    ``evict()`` after ``optimizer.step`` copies every state tensor to its pinned mirror on the side stream and then
    releases the device storage (the tensor objects the optimizer holds stay the same, their storage shrinks to
    zero bytes); ``fetch()`` before the next step gives the storage back and refills it. With ``nvme_dir`` the
    mirrors are also written to one file per tensor and read back from there, which is what survives when the host
    memory is needed for something else. Tensors whose storage cannot be resized (slices of a symmetric arena)
    are left where they are.

    reference: ``src/distributed/zero_sharding.zig:183-247`` (``offloadToCPU`` / ``offloadToNVMe`` /
    ``loadFromNVMe``), YAML ``runtime.cpu_offload``, ``runtime.nvme_offload``, ``runtime.nvme_path``.
    """

    def __init__(self, tensors: Dict[str, torch.Tensor], device: torch.device, nvme_dir: Optional[str] = None):
        self.host = HostOffloader(device)
        self.nvme = NvmeStore(nvme_dir) if nvme_dir else None
        self.tensors: Dict[str, torch.Tensor] = {}
        self.nbytes: Dict[str, int] = {}
        for name, t in tensors.items():
            st = t.untyped_storage()
            # only whole, privately owned storages can be released and re-created
            if t.is_contiguous() and t.storage_offset() == 0 and st.nbytes() == t.numel() * t.element_size() and st.resizable():
                self.tensors[name] = t
                self.nbytes[name] = st.nbytes()
        self.resident = True

    def evict(self) -> None:
        if not self.resident:
            return
        for name, t in self.tensors.items():
            self.host.offload(name, t)
        self.host.synchronize()                       # the copies have left the device before its memory is released
        for name, t in self.tensors.items():
            if self.nvme is not None:
                self.nvme.write(name, self.host.mirrors[name])
            t.untyped_storage().resize_(0)
        if self.nvme is not None:
            self.nvme.flush()
        self.resident = False

    def fetch(self) -> None:
        if self.resident:
            return
        for name, t in self.tensors.items():
            t.untyped_storage().resize_(self.nbytes[name])
            if self.nvme is not None:
                self.nvme.read(name, self.host.mirrors[name]).wait()
            self.host.prefetch(name, t)
        self.host.wait()
        self.resident = True

    def device_bytes(self) -> int:
        return sum(t.untyped_storage().nbytes() for t in self.tensors.values())

    def close(self) -> None:
        self.fetch()
        if self.nvme is not None:
            self.nvme.close()


class PinnedPool:
    """One page-locked host slab handed out as aligned tensor views by a bump pointer (``reset`` frees everything at
    once): staging buffers for host <-> device copies without a ``cudaHostAlloc`` per tensor. On a machine without CUDA
    the slab is ordinary host memory.

    reference: ``src/memory.zig:73-106`` (``PinnedMemoryPool``: bump allocation out of one pinned buffer).
    """

    ALIGN = 256

    def __init__(self, nbytes: int, pin: Optional[bool] = None):
        self.capacity = (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.slab = torch.empty(self.capacity, dtype=torch.uint8)
        if torch.cuda.is_available() if pin is None else pin:
            self.slab = self.slab.pin_memory()
        self.offset = 0
        self.peak = 0

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self.offset + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if start + nbytes > self.capacity:
            raise MemoryError(f"pinned pool exhausted: {nbytes} bytes requested, {self.capacity - start} left of {self.capacity}")
        self.offset = start + nbytes
        self.peak = max(self.peak, self.offset)
        return self.slab[start:start + nbytes].view(dtype).view(*shape)

    def reset(self) -> None:
        self.offset = 0

    def bytes_free(self) -> int:
        return self.capacity - self.offset
