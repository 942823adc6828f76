"""ctypes binding of ``libsynaptik_cuda.so``: the Python twin of the Java ``CudaNativeApi``.

Mirrors the reference's native seam (modules/backend/metal/.../MetalNativeApi.java:3648-3708):
the library path is explicit, every symbol is required, the ABI version is probed first, every
status other than 0 raises ``NativeFailure(operation, status)`` and nothing is retried or routed
elsewhere.  There is no CPU path behind this module: without the built library it raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Iterable, Sequence

import numpy as np

ABI_VERSION = 1
_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIBRARY = os.path.join(_HERE, "lib", "libsynaptik_cuda.so")

STATUS_NAMES = {
    0: "OK", 1: "INVALID_ARGUMENT", 2: "NO_DEVICE", 3: "NO_STREAM", 4: "ALLOCATION_FAILED",
    5: "RANGE_OUT_OF_BOUNDS", 6: "COPY_FAILED", 7: "INTERNAL_ERROR", 8: "UNSUPPORTED_SHAPE",
    9: "GRAPH_COMPILATION_FAILED", 10: "INCOMPATIBLE_RESOURCE", 11: "EXECUTION_FAILED",
    12: "KERNEL_COMPILATION_FAILED", 13: "UNSUPPORTED_OPERATION", 14: "TIMEOUT", 15: "COMM_FAILED",
}

# every symbol include/synaptik_cuda.h declares; all are required at load time
SYMBOLS = [
    "synaptik_cuda_abi_version", "synaptik_cuda_context_create", "synaptik_cuda_context_release",
    "synaptik_cuda_context_set_option", "synaptik_cuda_context_synchronize",
    "synaptik_cuda_context_timer_start", "synaptik_cuda_context_timer_stop", "synaptik_cuda_context_wait_probe",
    "synaptik_cuda_context_occupy",
    "synaptik_cuda_executable_describe", "synaptik_cuda_executable_step_timings",
    "synaptik_cuda_buffer_create", "synaptik_cuda_buffer_release", "synaptik_cuda_buffer_upload",
    "synaptik_cuda_buffer_download", "synaptik_cuda_buffer_upload_canonical",
    "synaptik_cuda_buffer_download_canonical", "synaptik_cuda_buffer_upload_async",
    "synaptik_cuda_buffer_download_async", "synaptik_cuda_buffer_prefetch", "synaptik_cuda_buffer_device_pointer",
    "synaptik_cuda_host_alloc", "synaptik_cuda_host_free",
    "synaptik_cuda_executable_create", "synaptik_cuda_executable_release", "synaptik_cuda_executable_run",
    "synaptik_cuda_executable_enqueue", "synaptik_cuda_executable_finish", "synaptik_cuda_program_describe",
    "synaptik_cuda_executable_last_timing", "synaptik_cuda_executable_launch_count",
    "synaptik_cuda_optimizer_create", "synaptik_cuda_optimizer_release", "synaptik_cuda_optimizer_step",
    "synaptik_cuda_optimizer_step_enqueue", "synaptik_cuda_optimizer_finish", "synaptik_cuda_optimizer_steps",
    "synaptik_cuda_optimizer_download_state", "synaptik_cuda_optimizer_upload_state",
    "synaptik_cuda_optimizer_run", "synaptik_cuda_optimizer_run_enqueue", "synaptik_cuda_optimizer_zero_grad",
    "synaptik_cuda_optimizer_accumulated_runs", "synaptik_cuda_optimizer_download_state_canonical",
    "synaptik_cuda_optimizer_upload_state_canonical", "synaptik_cuda_optimizer_set_progress",
    "synaptik_cuda_comm_unique_id", "synaptik_cuda_comm_create", "synaptik_cuda_comm_release",
    "synaptik_cuda_comm_allreduce_sum_f32", "synaptik_cuda_executable_attach_comm",
    "synaptik_cuda_column_sums_no_alloc",
]


class NativeFailure(RuntimeError):
    """A native entry point returned a non-zero status (MetalNativeApi.NativeFailure)."""

    def __init__(self, operation: str, status: int):
        self.operation = operation
        self.status = status
        super().__init__(f"{operation} failed with status {status} ({STATUS_NAMES.get(status, 'UNKNOWN')})")


_library = None


def library(path: str | None = None) -> ctypes.CDLL:
    """Loads the shim (once).  Raises if it is missing, lacks a symbol or reports another ABI."""
    global _library
    if _library is not None and path is None:
        return _library
    path = path or os.environ.get("SYNAPTIK_CUDA_LIBRARY") or DEFAULT_LIBRARY
    if not os.path.isabs(path):
        raise ValueError("the native library path must be absolute")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} is missing: build it with `python -m synaptik_b200.build` "
                                "(there is no CPU fallback)")
    lib = ctypes.CDLL(path)
    for name in SYMBOLS:
        getattr(lib, name).restype = ctypes.c_int32
    lib.synaptik_cuda_abi_version.restype = ctypes.c_uint32
    if lib.synaptik_cuda_abi_version() != ABI_VERSION:
        raise RuntimeError(f"ABI version {lib.synaptik_cuda_abi_version()} != {ABI_VERSION}")
    _library = lib
    return lib


def _check(operation: str, status: int) -> None:
    if status != 0:
        raise NativeFailure(operation, int(status))


class Context:
    def __init__(self, device_ordinal: int = 0):
        self._h = ctypes.c_void_p()
        self.device_ordinal = device_ordinal
        _check("context_create", library().synaptik_cuda_context_create(ctypes.c_int32(device_ordinal), ctypes.byref(self._h)))

    def set_option(self, name: str, value: int) -> None:
        _check("context_set_option", library().synaptik_cuda_context_set_option(self._h, name.encode(), ctypes.c_int64(value)))

    def synchronize(self) -> None:
        _check("context_synchronize", library().synaptik_cuda_context_synchronize(self._h))

    def timer_start(self) -> None:
        _check("context_timer_start", library().synaptik_cuda_context_timer_start(self._h))

    def timer_stop(self) -> float:
        ms = ctypes.c_double()
        _check("context_timer_stop", library().synaptik_cuda_context_timer_stop(self._h, ctypes.byref(ms)))
        return float(ms.value)

    def wait_probe(self, limit_microseconds: int) -> None:
        """Runs the give-up path of the device-side bounded waits; always raises NativeFailure(14)."""
        _check("context_wait_probe", library().synaptik_cuda_context_wait_probe(self._h, ctypes.c_uint64(limit_microseconds)))

    def occupy(self, blocks: int, hold_microseconds: int) -> None:
        """Enqueues `blocks` blocks on the communication stream that each hold one SM for the given time."""
        _check("context_occupy", library().synaptik_cuda_context_occupy(self._h, ctypes.c_int32(blocks), ctypes.c_uint64(hold_microseconds)))

    def buffer(self, nbytes: int) -> "Buffer":
        return Buffer(self, nbytes)

    def upload(self, array: np.ndarray) -> "Buffer":
        array = np.ascontiguousarray(array)
        b = Buffer(self, array.nbytes)
        b.upload(array)
        return b

    def close(self) -> None:
        if self._h:
            _check("context_release", library().synaptik_cuda_context_release(self._h))
            self._h = ctypes.c_void_p()


class Buffer:
    def __init__(self, context: Context, nbytes: int):
        self.context = context
        self.nbytes = int(nbytes)
        self._h = ctypes.c_void_p()
        _check("buffer_create", library().synaptik_cuda_buffer_create(context._h, ctypes.c_uint64(self.nbytes), ctypes.byref(self._h)))

    def upload(self, array: np.ndarray, offset: int = 0) -> None:
        array = np.ascontiguousarray(array)
        _check("buffer_upload", library().synaptik_cuda_buffer_upload(
            self._h, ctypes.c_uint64(offset), array.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(array.nbytes)))

    def download(self, dtype, shape, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        _check("buffer_download", library().synaptik_cuda_buffer_download(
            self._h, ctypes.c_uint64(offset), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(out.nbytes)))
        return out

    def upload_canonical(self, data: bytes, element_bytes: int, offset: int = 0) -> None:
        _check("buffer_upload_canonical", library().synaptik_cuda_buffer_upload_canonical(
            self._h, ctypes.c_uint64(offset), data, ctypes.c_uint64(len(data)), ctypes.c_uint32(element_bytes)))

    def download_canonical(self, nbytes: int, element_bytes: int, offset: int = 0) -> bytes:
        out = ctypes.create_string_buffer(nbytes)
        _check("buffer_download_canonical", library().synaptik_cuda_buffer_download_canonical(
            self._h, ctypes.c_uint64(offset), out, ctypes.c_uint64(nbytes), ctypes.c_uint32(element_bytes)))
        return out.raw

    def upload_async(self, pointer: int, nbytes: int, offset: int = 0) -> None:
        _check("buffer_upload_async", library().synaptik_cuda_buffer_upload_async(
            self._h, ctypes.c_uint64(offset), ctypes.c_void_p(pointer), ctypes.c_uint64(nbytes)))

    def prefetch(self, pointer: int, nbytes: int, offset: int = 0) -> None:
        """Upload from pinned memory on the copy stream, overlapping the compute stream's work."""
        _check("buffer_prefetch", library().synaptik_cuda_buffer_prefetch(
            self._h, ctypes.c_uint64(offset), ctypes.c_void_p(pointer), ctypes.c_uint64(nbytes)))

    def download_async(self, pointer: int, nbytes: int, offset: int = 0) -> None:
        _check("buffer_download_async", library().synaptik_cuda_buffer_download_async(
            self._h, ctypes.c_uint64(offset), ctypes.c_void_p(pointer), ctypes.c_uint64(nbytes)))

    def device_pointer(self) -> int:
        address = ctypes.c_uint64()
        size = ctypes.c_uint64()
        _check("buffer_device_pointer", library().synaptik_cuda_buffer_device_pointer(self._h, ctypes.byref(address), ctypes.byref(size)))
        return int(address.value)

    def close(self) -> None:
        if self._h:
            _check("buffer_release", library().synaptik_cuda_buffer_release(self._h))
            self._h = ctypes.c_void_p()


class PinnedArray:
    """Page-locked host memory viewed as a numpy array (the staging side of ``borrow``)."""

    def __init__(self, shape, dtype):
        self.shape = tuple(shape)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        self._p = ctypes.c_void_p()
        _check("host_alloc", library().synaptik_cuda_host_alloc(ctypes.c_uint64(self.nbytes), ctypes.byref(self._p)))
        raw = (ctypes.c_uint8 * max(self.nbytes, 1)).from_address(self._p.value)
        self.array = np.frombuffer(raw, dtype=self.dtype, count=int(np.prod(self.shape))).reshape(self.shape)

    @property
    def pointer(self) -> int:
        return int(self._p.value)

    def close(self) -> None:
        if self._p:
            self.array = None
            _check("host_free", library().synaptik_cuda_host_free(self._p))
            self._p = ctypes.c_void_p()


def _handles(buffers: Sequence[Buffer]):
    array = (ctypes.c_void_p * max(len(buffers), 1))()
    for i, b in enumerate(buffers):
        array[i] = b._h
    return array


def describe(image: bytes) -> str:
    """Lowered launch plan of a program image, one line per launch.  Needs no GPU."""
    required = ctypes.c_uint64()
    status = library().synaptik_cuda_program_describe(image, ctypes.c_uint32(len(image)), None, ctypes.c_uint64(0), ctypes.byref(required))
    if status != 1 or required.value == 0:      # INVALID_ARGUMENT with the size filled in is the size probe
        _check("program_describe", status if status else 7)
    text = ctypes.create_string_buffer(int(required.value))
    _check("program_describe", library().synaptik_cuda_program_describe(image, ctypes.c_uint32(len(image)), text, required, None))
    return text.value.decode()


class Executable:
    def __init__(self, context: Context, image: bytes):
        self.context = context
        self._h = ctypes.c_void_p()
        _check("executable_create", library().synaptik_cuda_executable_create(context._h, image, ctypes.c_uint32(len(image)), ctypes.byref(self._h)))

    def run(self, inputs: Sequence[Buffer], outputs: Sequence[Buffer]) -> None:
        _check("executable_run", library().synaptik_cuda_executable_run(
            self._h, ctypes.c_int32(len(inputs)), _handles(inputs), ctypes.c_int32(len(outputs)), _handles(outputs)))

    def enqueue(self, inputs: Sequence[Buffer], outputs: Sequence[Buffer]) -> None:
        _check("executable_enqueue", library().synaptik_cuda_executable_enqueue(
            self._h, ctypes.c_int32(len(inputs)), _handles(inputs), ctypes.c_int32(len(outputs)), _handles(outputs)))

    def finish(self) -> None:
        _check("executable_finish", library().synaptik_cuda_executable_finish(self._h))

    def last_timing_ms(self) -> float:
        ms = ctypes.c_double()
        _check("executable_last_timing", library().synaptik_cuda_executable_last_timing(self._h, ctypes.byref(ms)))
        return float(ms.value)

    def describe(self) -> str:
        required = ctypes.c_uint64()
        library().synaptik_cuda_executable_describe(self._h, None, ctypes.c_uint64(0), ctypes.byref(required))
        text = ctypes.create_string_buffer(int(required.value))
        _check("executable_describe", library().synaptik_cuda_executable_describe(self._h, text, required, None))
        return text.value.decode()

    def step_timings_ms(self):
        count = ctypes.c_uint64()
        library().synaptik_cuda_executable_step_timings(self._h, None, ctypes.c_uint64(0), ctypes.byref(count))
        out = (ctypes.c_double * max(int(count.value), 1))()
        _check("executable_step_timings", library().synaptik_cuda_executable_step_timings(self._h, out, count, ctypes.byref(count)))
        return [float(out[i]) for i in range(int(count.value))]

    def launch_count(self) -> int:
        n = ctypes.c_uint64()
        _check("executable_launch_count", library().synaptik_cuda_executable_launch_count(self._h, ctypes.byref(n)))
        return int(n.value)

    def attach_comm(self, comm: "Comm | None", output_indices: Iterable[int] = ()) -> None:
        indices = list(output_indices)
        array = (ctypes.c_int32 * max(len(indices), 1))(*indices)
        _check("executable_attach_comm", library().synaptik_cuda_executable_attach_comm(
            self._h, comm._h if comm is not None else None, ctypes.c_int32(len(indices)), array))

    def close(self) -> None:
        if self._h:
            _check("executable_release", library().synaptik_cuda_executable_release(self._h))
            self._h = ctypes.c_void_p()


SGD, ADAM, ADAMW = 0, 1, 2


class Optimizer:
    def __init__(self, context: Context, kind: int, hyper: Sequence[float], parameters: Sequence[Buffer], counts: Sequence[int]):
        self.context = context
        self._h = ctypes.c_void_p()
        h = (ctypes.c_double * 5)(*hyper)
        c = (ctypes.c_uint64 * len(counts))(*counts)
        _check("optimizer_create", library().synaptik_cuda_optimizer_create(
            context._h, ctypes.c_int32(kind), h, ctypes.c_int32(5), ctypes.c_int32(len(parameters)), _handles(parameters), c, ctypes.byref(self._h)))
        self.counts = list(counts)

    def step(self, gradients: Sequence[Buffer]) -> None:
        _check("optimizer_step", library().synaptik_cuda_optimizer_step(self._h, ctypes.c_int32(len(gradients)), _handles(gradients)))

    def step_enqueue(self, gradients: Sequence[Buffer]) -> None:
        _check("optimizer_step_enqueue", library().synaptik_cuda_optimizer_step_enqueue(self._h, ctypes.c_int32(len(gradients)), _handles(gradients)))

    def finish(self) -> None:
        _check("optimizer_finish", library().synaptik_cuda_optimizer_finish(self._h))

    RESET_AND_STEP, ACCUMULATE, ACCUMULATE_AND_STEP = 0, 1, 2

    def run(self, gradient_mode: int, gradients: Sequence[Buffer]) -> None:
        """One training run's optimizer side under a GradientMode (TrainingSession.runValues)."""
        _check("optimizer_run", library().synaptik_cuda_optimizer_run(
            self._h, ctypes.c_int32(gradient_mode), ctypes.c_int32(len(gradients)), _handles(gradients)))

    def zero_grad(self) -> None:
        _check("optimizer_zero_grad", library().synaptik_cuda_optimizer_zero_grad(self._h))

    def accumulated_runs(self) -> int:
        n = ctypes.c_uint64()
        _check("optimizer_accumulated_runs", library().synaptik_cuda_optimizer_accumulated_runs(self._h, ctypes.byref(n)))
        return int(n.value)

    def state_canonical(self, index: int, slot: int) -> bytes:
        """Big-endian FLOAT32 bytes of one optimizer-width array, as TrainingState stores them."""
        out = ctypes.create_string_buffer(self.counts[index] * 4)
        _check("optimizer_download_state_canonical", library().synaptik_cuda_optimizer_download_state_canonical(
            self._h, ctypes.c_int32(index), ctypes.c_int32(slot), out, ctypes.c_uint64(self.counts[index] * 4)))
        return out.raw

    def restore_canonical(self, index: int, slot: int, data: bytes) -> None:
        _check("optimizer_upload_state_canonical", library().synaptik_cuda_optimizer_upload_state_canonical(
            self._h, ctypes.c_int32(index), ctypes.c_int32(slot), data, ctypes.c_uint64(len(data))))

    def set_progress(self, completed_steps: int, accumulated_runs: int) -> None:
        _check("optimizer_set_progress", library().synaptik_cuda_optimizer_set_progress(
            self._h, ctypes.c_uint64(completed_steps), ctypes.c_uint64(accumulated_runs)))

    def steps(self) -> int:
        n = ctypes.c_uint64()
        _check("optimizer_steps", library().synaptik_cuda_optimizer_steps(self._h, ctypes.byref(n)))
        return int(n.value)

    def state(self, index: int, slot: int) -> np.ndarray:
        out = np.empty(self.counts[index], dtype=np.float32)
        _check("optimizer_download_state", library().synaptik_cuda_optimizer_download_state(
            self._h, ctypes.c_int32(index), ctypes.c_int32(slot), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(out.nbytes)))
        return out

    def restore(self, index: int, slot: int, values: np.ndarray, completed_steps: int) -> None:
        values = np.ascontiguousarray(values, dtype=np.float32)
        _check("optimizer_upload_state", library().synaptik_cuda_optimizer_upload_state(
            self._h, ctypes.c_int32(index), ctypes.c_int32(slot), values.ctypes.data_as(ctypes.c_void_p),
            ctypes.c_uint64(values.nbytes), ctypes.c_uint64(completed_steps)))

    def close(self) -> None:
        if self._h:
            _check("optimizer_release", library().synaptik_cuda_optimizer_release(self._h))
            self._h = ctypes.c_void_p()


def column_sums_no_alloc(context: Context, source: Buffer, rows: int, cols: int, destination: Buffer) -> None:
    """Column sums of a dense [rows, cols] FP32 buffer into `destination`, for callers that must not
    allocate: the scratch is a fixed array inside the library (see include/synaptik_cuda.h)."""
    _check("column_sums_no_alloc", library().synaptik_cuda_column_sums_no_alloc(
        context._h, source._h, ctypes.c_uint64(rows), ctypes.c_uint64(cols), destination._h))


def comm_unique_id() -> bytes:
    out = (ctypes.c_uint8 * 128)()
    _check("comm_unique_id", library().synaptik_cuda_comm_unique_id(out))
    return bytes(out)


class Comm:
    def __init__(self, context: Context, world_size: int, rank: int, unique_id: bytes):
        self.context = context
        self.world_size, self.rank = world_size, rank
        self._h = ctypes.c_void_p()
        _check("comm_create", library().synaptik_cuda_comm_create(
            context._h, ctypes.c_int32(world_size), ctypes.c_int32(rank), unique_id, ctypes.byref(self._h)))

    def allreduce_sum(self, buffer: Buffer, count: int, offset: int = 0) -> None:
        _check("comm_allreduce_sum_f32", library().synaptik_cuda_comm_allreduce_sum_f32(
            self._h, buffer._h, ctypes.c_uint64(offset), ctypes.c_uint64(count)))

    def close(self) -> None:
        if self._h:
            _check("comm_release", library().synaptik_cuda_comm_release(self._h))
            self._h = ctypes.c_void_p()
