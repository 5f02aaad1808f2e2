"""ctypes binding of the C ABI in include/b200_gemm.h.

The Python names mirror the reference's host interface: ``gemm`` is ``gpu_gemm(GemmParams)``
(matmul_h100.cu.jinja:927-985), ``run_kernel`` is ``runKernel`` (matmul_h100_optimal.cu:32-59),
``reference_gpu_gemm`` is the naive device GEMM of reference.h:78-90, and ``GemmConfig`` carries
the template variables of matmul_h100.cu.jinja:9-14. Tensors are torch CUDA tensors used purely
as device-memory handles; all arithmetic happens in the shared library's kernels.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import os

# B200_GEMM_LIBRARY points the binding at another build of the same C ABI (A/B comparisons).
_LIB_PATH = Path(os.environ.get("B200_GEMM_LIBRARY") or
                 Path(__file__).resolve().parent / "lib" / "libb200gemm.so")
_lib = None

STATUS_OK = 0
STATUS_INVALID_ARG = 1
STATUS_UNSUPPORTED_CFG = 2
STATUS_SMEM = 3
STATUS_WORKSPACE = 4
STATUS_CUDA = 5
STATUS_DEVICE_TIMEOUT = 6
STATUS_STATIC_SCRATCH = 8


class GemmError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b200_gemm status {status}: {message}")
        self.status = status


class _Cfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "block_m", "block_n", "block_k", "stages", "cluster_m", "cluster_n", "sched", "split_k",
        "raster", "group", "c_col_major", "max_ctas", "epilogue", "swap_ab")]


@dataclass
class GemmConfig:
    """Tunable surface; field meanings are documented in include/b200_gemm.h."""
    block_m: int = 128
    block_n: int = 256
    block_k: int = 64
    stages: int = 0
    cluster_m: int = 2
    cluster_n: int = 1
    sched: int = 0
    split_k: int = 0
    raster: int = 0
    group: int = 0
    c_col_major: int = 0
    max_ctas: int = 0
    epilogue: int = 0
    swap_ab: int = 0

    def _c(self) -> _Cfg:
        return _Cfg(self.block_m, self.block_n, self.block_k, self.stages, self.cluster_m,
                    self.cluster_n, self.sched, self.split_k, self.raster, self.group,
                    self.c_col_major, self.max_ctas, self.epilogue, self.swap_ab)


def library() -> ctypes.CDLL:
    """Loads libb200gemm.so; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise GemmError(-1, f"{_LIB_PATH} is missing: run `python -m h100_gemm_b200.build`")
    lib = ctypes.CDLL(str(_LIB_PATH))
    vp, ci, cf, ll, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_size_t
    cfgp = ctypes.POINTER(_Cfg)
    lib.b200_gemm_bf16.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf, cfgp, vp, sz, vp]
    lib.b200_gemm_bf16.restype = ci
    if hasattr(lib, "b200_gemm_f16"):
        lib.b200_gemm_f16.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf, cfgp, vp, sz, vp]
        lib.b200_gemm_f16.restype = ci
        lib.b200_reference_gpu_gemm_f16.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf, vp]
        lib.b200_reference_gpu_gemm_f16.restype = ci
    lib.b200_gemm_batched_bf16.argtypes = [ci, ci, ci, ci, vp, ll, vp, ll, vp, ll, cf, cf, cfgp, vp, sz, vp]
    lib.b200_gemm_batched_bf16.restype = ci
    lib.b200_gemm_workspace_bytes.argtypes = [ci, ci, ci, ci, cfgp]
    lib.b200_gemm_workspace_bytes.restype = sz
    lib.b200_gemm_default_cfg.argtypes = [ci, ci, ci, ci, cfgp]
    lib.b200_gemm_default_cfg.restype = ci
    lib.b200_run_kernel.argtypes = [ci, ci, ci, vp, vp, vp, vp]
    lib.b200_run_kernel.restype = ci
    lib.b200_gemm_bf16_host.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf, cfgp]
    lib.b200_gemm_bf16_host.restype = ci
    lib.b200_gemm_bf16_host_copies_only.argtypes = [ci, ci, ci, vp, vp, vp]
    lib.b200_gemm_bf16_host_copies_only.restype = ci
    lib.b200_gemm_host_release.argtypes = []
    lib.b200_gemm_host_release.restype = None
    lib.b200_reference_gpu_gemm_bf16.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf, vp]
    lib.b200_reference_gpu_gemm_bf16.restype = ci
    lib.b200_gemm_last_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint * 4)]
    lib.b200_gemm_last_device_status.restype = ci
    if hasattr(lib, "b200_gemm_set_profile_buffer"):  # absent from older builds of the ABI
        lib.b200_gemm_set_profile_buffer.argtypes = [vp, sz]
        lib.b200_gemm_set_profile_buffer.restype = ci
    lib.b200_gemm_selftest_bounded_wait.argtypes = [ll]
    lib.b200_gemm_selftest_bounded_wait.restype = ci
    if hasattr(lib, "b200_gemm_bf16_fixed_scratch"):
        lib.b200_gemm_bf16_fixed_scratch.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf, vp]
        lib.b200_gemm_bf16_fixed_scratch.restype = ci
        lib.b200_gemm_fixed_scratch_cfg.argtypes = [ci, ci, ci, cfgp]
        lib.b200_gemm_fixed_scratch_cfg.restype = ci
    if hasattr(lib, "b200_gemm_bf16_gather"):
        lib.b200_gemm_bf16_gather.argtypes = [ci, ci, ci, vp, vp, ctypes.POINTER(vp), ci, ci, cfgp, vp]
        lib.b200_gemm_bf16_gather.restype = ci
        lib.b200_peer_alloc.argtypes = [sz, ctypes.POINTER(vp)]
        lib.b200_peer_free.argtypes = [vp]
        lib.b200_peer_export.argtypes = [vp, ctypes.c_char_p]
        lib.b200_peer_import.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        lib.b200_peer_close.argtypes = [vp]
        for f in (lib.b200_peer_alloc, lib.b200_peer_free, lib.b200_peer_export, lib.b200_peer_import,
                  lib.b200_peer_close):
            f.restype = ci
    if hasattr(lib, "b200_mgemm_create"):
        lib.b200_mgemm_create.argtypes = [ctypes.POINTER(vp), ci, ctypes.POINTER(ci), ci, ci, ci, ci]
        lib.b200_mgemm_buffers.argtypes = [vp, ci, ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp)]
        lib.b200_mgemm_run.argtypes = [vp]
        lib.b200_mgemm_sync.argtypes = [vp, ctypes.POINTER(cf)]
        lib.b200_mgemm_destroy.argtypes = [vp]
        for f in (lib.b200_mgemm_create, lib.b200_mgemm_buffers, lib.b200_mgemm_run, lib.b200_mgemm_sync,
                  lib.b200_mgemm_destroy):
            f.restype = ci
    lib.b200_gemm_tuning_load.argtypes = [ctypes.c_char_p]
    lib.b200_gemm_tuning_load.restype = ci
    lib.b200_gemm_tuning_add.argtypes = [ci, ci, ci, ci, cfgp]
    lib.b200_gemm_tuning_add.restype = ci
    lib.b200_gemm_tuning_clear.argtypes = []
    lib.b200_gemm_tuning_clear.restype = None
    lib.b200_gemm_tuning_size.argtypes = []
    lib.b200_gemm_tuning_size.restype = ci
    lib.b200_gemm_heuristic_cfg.argtypes = [ci, ci, ci, ci, cfgp]
    lib.b200_gemm_heuristic_cfg.restype = ci
    lib.b200_gemm_heuristic_cfg_for_sms.argtypes = [ci, ci, ci, ci, ci, cfgp]
    lib.b200_gemm_heuristic_cfg_for_sms.restype = ci
    lib.b200_gemm_strerror.argtypes = [ci]
    lib.b200_gemm_strerror.restype = ctypes.c_char_p
    lib.b200_gemm_last_cuda_error.argtypes = []
    lib.b200_gemm_last_cuda_error.restype = ci
    lib.b200_gemm_sm_count.argtypes = []
    lib.b200_gemm_sm_count.restype = ci
    _lib = lib
    return lib


def _check(status: int) -> None:
    if status != STATUS_OK:
        lib = library()
        msg = lib.b200_gemm_strerror(status).decode()
        if status == STATUS_CUDA:
            msg += f" (CUDA error {lib.b200_gemm_last_cuda_error()})"
        raise GemmError(status, msg)


def _cfg_ptr(cfg: Optional[GemmConfig]):
    if cfg is None:
        return None, None
    c = cfg._c()
    return c, ctypes.byref(c)


def _stream_ptr(stream) -> Optional[int]:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream or None
    return getattr(stream, "cuda_stream", stream) or None


def _require_cuda_bf16(t, name: str, ndim: int, dtype=None):
    import torch
    dtype = dtype or torch.bfloat16
    if not t.is_cuda:
        raise GemmError(STATUS_INVALID_ARG, f"{name} must be a CUDA tensor (no CPU fallback exists)")
    if t.dtype != dtype or t.dim() != ndim or not t.is_contiguous():
        raise GemmError(STATUS_INVALID_ARG, f"{name} must be a contiguous {ndim}-D {dtype} tensor")


def workspace_bytes(batch: int, M: int, N: int, K: int, cfg: Optional[GemmConfig] = None) -> int:
    keep, p = _cfg_ptr(cfg)
    return int(library().b200_gemm_workspace_bytes(batch, M, N, K, p))


def default_config(batch: int, M: int, N: int, K: int) -> GemmConfig:
    c = _Cfg()
    _check(library().b200_gemm_default_cfg(batch, M, N, K, ctypes.byref(c)))
    return GemmConfig(**{n: getattr(c, n) for n, _ in _Cfg._fields_})


def heuristic_config(batch: int, M: int, N: int, K: int) -> GemmConfig:
    """The built-in choice for a shape, ignoring the tuning table."""
    c = _Cfg()
    _check(library().b200_gemm_heuristic_cfg(batch, M, N, K, ctypes.byref(c)))
    return GemmConfig(**{n: getattr(c, n) for n, _ in _Cfg._fields_})


def heuristic_config_for_sms(batch: int, M: int, N: int, K: int, sm_count: int) -> GemmConfig:
    """The built-in choice for a device with `sm_count` multiprocessors."""
    c = _Cfg()
    _check(library().b200_gemm_heuristic_cfg_for_sms(batch, M, N, K, sm_count, ctypes.byref(c)))
    return GemmConfig(**{n: getattr(c, n) for n, _ in _Cfg._fields_})


def tuning_load(path) -> int:
    """Adds the entries of a tuning-table file (the format `gemm_tuner.py --table` writes) to the
    table that ``cfg=None`` calls consult before the heuristic; returns how many were read."""
    n = int(library().b200_gemm_tuning_load(str(path).encode()))
    if n < 0:
        raise GemmError(-n, f"tuning table {path}: {library().b200_gemm_strerror(-n).decode()}")
    return n


def tuning_add(M: int, N: int, K: int, cfg: GemmConfig, batch: int = 1) -> None:
    _check(library().b200_gemm_tuning_add(batch, M, N, K, ctypes.byref(cfg._c())))


def tuning_clear() -> None:
    library().b200_gemm_tuning_clear()


def tuning_size() -> int:
    return int(library().b200_gemm_tuning_size())


def _workspace(nbytes: int, workspace, device):
    import torch
    if nbytes == 0:
        return None, 0
    if workspace is None:
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
    if workspace.numel() * workspace.element_size() < nbytes:
        raise GemmError(STATUS_WORKSPACE, f"workspace needs {nbytes} bytes")
    return workspace, workspace.numel() * workspace.element_size()


def gemm(a, b, out=None, alpha: float = 1.0, beta: float = 0.0, cfg: Optional[GemmConfig] = None,
         workspace=None, stream=None):
    """out[M,N] = (bf16)(a[M,K] @ b[N,K]^T * alpha + beta) on the current CUDA device.

    With ``cfg.c_col_major`` the result is written column-major: ``out`` must then have shape
    [N, M] (it holds C^T row-major), as matmulKernel of the reference does (matmul_utils.cuh:529).
    """
    import torch
    dtype = torch.float16 if a.dtype == torch.float16 else torch.bfloat16  # fp16 -> b200_gemm_f16
    _require_cuda_bf16(a, "a", 2, dtype)
    _require_cuda_bf16(b, "b", 2, dtype)
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb:
        raise GemmError(STATUS_INVALID_ARG, "a and b disagree on K")
    col_major = bool(cfg is not None and cfg.c_col_major)
    shape = (N, M) if col_major else (M, N)
    if out is None:
        out = torch.empty(shape, dtype=dtype, device=a.device)
    _require_cuda_bf16(out, "out", 2, dtype)
    if tuple(out.shape) != shape:
        raise GemmError(STATUS_INVALID_ARG, f"out must have shape {shape}")
    ws, ws_bytes = _workspace(workspace_bytes(1, M, N, K, cfg), workspace, a.device)
    keep, p = _cfg_ptr(cfg)
    fn = library().b200_gemm_f16 if dtype == torch.float16 else library().b200_gemm_bf16
    _check(fn(M, N, K, a.data_ptr(), b.data_ptr(), out.data_ptr(), alpha, beta,
                                    p, ws.data_ptr() if ws is not None else None, ws_bytes,
                                    _stream_ptr(stream)))
    return out


def gemm_fixed_scratch(a, b, out=None, alpha: float = 1.0, beta: float = 0.0, stream=None):
    """out[M,N] = a @ b^T for M <= 128 without any device allocation by the library or a workspace
    from the caller (b200_gemm_bf16_fixed_scratch; see include/b200_gemm.h for who needs this and
    the limits). `out` must be supplied by callers that themselves may not allocate."""
    import torch
    _require_cuda_bf16(a, "a", 2)
    _require_cuda_bf16(b, "b", 2)
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb:
        raise GemmError(STATUS_INVALID_ARG, "a and b disagree on K")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    _require_cuda_bf16(out, "out", 2)
    _check(library().b200_gemm_bf16_fixed_scratch(M, N, K, a.data_ptr(), b.data_ptr(), out.data_ptr(), alpha,
                                                  beta, _stream_ptr(stream)))
    return out


class DeviceBuffer:
    """A cudaMalloc allocation other processes of the node can map (CUDA IPC), viewable as a torch
    tensor. Used for the per-rank copies of C that the fused gather GEMM writes into."""

    def __init__(self, nbytes: int):
        self.nbytes = nbytes
        p = ctypes.c_void_p()
        _check(library().b200_peer_alloc(nbytes, ctypes.byref(p)))
        self.ptr = p.value
        self._imported = False

    @classmethod
    def from_handle(cls, handle: bytes, nbytes: int) -> "DeviceBuffer":
        self = cls.__new__(cls)
        p = ctypes.c_void_p()
        _check(library().b200_peer_import(handle, ctypes.byref(p)))
        self.ptr, self.nbytes, self._imported = p.value, nbytes, True
        return self

    def handle(self) -> bytes:
        buf = ctypes.create_string_buffer(64)
        _check(library().b200_peer_export(self.ptr, buf))
        return buf.raw

    def tensor(self, shape, dtype=None):
        """A torch view of the allocation (no copy)."""
        import torch
        dtype = dtype or torch.bfloat16
        n = 1
        for d in shape:
            n *= d

        class _Raw:
            pass

        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (n,), "typestr": "<i2", "data": (self.ptr, False), "version": 2}
        return torch.as_tensor(raw, device="cuda").view(dtype).view(*shape)

    def close(self) -> None:
        if self.ptr:
            if self._imported:
                library().b200_peer_close(self.ptr)
            else:
                library().b200_peer_free(self.ptr)
            self.ptr = None


class MultiGemm:
    """The single-process multi-GPU handle of the C ABI (b200_mgemm_*): rank p of `world` runs on
    ``devices[p]`` and owns A [M_shard, K], B [N, K] and C ([M_shard, N], or with ``gather`` the full
    [world * M_shard, N] that every rank's kernel writes into). Tensors returned by ``a``, ``b``
    and ``c`` are views of the handle's device buffers."""

    def __init__(self, world: int, M_shard: int, N: int, K: int, gather: bool = False, devices=None):
        self.world, self.M, self.N, self.K, self.gather = world, M_shard, N, K, bool(gather)
        self.devices = list(devices) if devices is not None else list(range(world))
        self._h = ctypes.c_void_p()
        arr = (ctypes.c_int * world)(*self.devices)
        _check(library().b200_mgemm_create(ctypes.byref(self._h), world, arr, M_shard, N, K, int(self.gather)))

    def _view(self, ptr: int, shape, device: int):
        import torch
        n = 1
        for d in shape:
            n *= d

        class _Raw:
            pass

        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (n,), "typestr": "<i2", "data": (ptr, False), "version": 2}
        with torch.cuda.device(device):
            return torch.as_tensor(raw, device=f"cuda:{device}").view(torch.bfloat16).view(*shape)

    def _buffers(self, rank: int):
        a, b, c = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        _check(library().b200_mgemm_buffers(self._h, rank, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)))
        return a.value, b.value, c.value

    def a(self, rank: int):
        return self._view(self._buffers(rank)[0], (self.M, self.K), self.devices[rank])

    def b(self, rank: int):
        return self._view(self._buffers(rank)[1], (self.N, self.K), self.devices[rank])

    def c(self, rank: int):
        rows = self.world * self.M if self.gather else self.M
        return self._view(self._buffers(rank)[2], (rows, self.N), self.devices[rank])

    def run(self) -> None:
        _check(library().b200_mgemm_run(self._h))

    def sync(self) -> float:
        """Waits for every device; returns the slowest device's time for the last run in ms."""
        ms = ctypes.c_float()
        _check(library().b200_mgemm_sync(self._h, ctypes.byref(ms)))
        return float(ms.value)

    def close(self) -> None:
        if self._h:
            library().b200_mgemm_destroy(self._h)
            self._h = ctypes.c_void_p()


def gemm_gather(a, b, c_all_ptrs, rank: int, cfg: Optional[GemmConfig] = None, stream=None) -> None:
    """Fused GEMM + all-gather (b200_gemm_bf16_gather): writes this rank's rows of C = a @ b^T into
    every pointer of `c_all_ptrs` (one full-C buffer per rank). The caller orders completion."""
    _require_cuda_bf16(a, "a", 2)
    _require_cuda_bf16(b, "b", 2)
    M, K = a.shape
    N = b.shape[0]
    world = len(c_all_ptrs)
    arr = (ctypes.c_void_p * world)(*c_all_ptrs)
    keep, p = _cfg_ptr(cfg)
    _check(library().b200_gemm_bf16_gather(M, N, K, a.data_ptr(), b.data_ptr(), arr, world, rank, p,
                                           _stream_ptr(stream)))


def gemm_batched(a, b, out=None, alpha: float = 1.0, beta: float = 0.0,
                 cfg: Optional[GemmConfig] = None, workspace=None, stream=None):
    """out[i] = a[i] @ b[i]^T for contiguous [batch, M, K] and [batch, N, K] tensors."""
    import torch
    _require_cuda_bf16(a, "a", 3)
    _require_cuda_bf16(b, "b", 3)
    batch, M, K = a.shape
    batch_b, N, Kb = b.shape
    if K != Kb or batch != batch_b:
        raise GemmError(STATUS_INVALID_ARG, "a and b disagree on batch or K")
    if out is None:
        out = torch.empty((batch, M, N), dtype=torch.bfloat16, device=a.device)
    _require_cuda_bf16(out, "out", 3)
    ws, ws_bytes = _workspace(workspace_bytes(batch, M, N, K, cfg), workspace, a.device)
    keep, p = _cfg_ptr(cfg)
    _check(library().b200_gemm_batched_bf16(
        batch, M, N, K, a.data_ptr(), M * K, b.data_ptr(), N * K, out.data_ptr(), M * N, alpha, beta, p,
        ws.data_ptr() if ws is not None else None, ws_bytes, _stream_ptr(stream)))
    return out


def run_kernel(a, b, out=None):
    """runKernel(M, N, K, A, B, C, DB): default configuration, column-major C, default stream.

    ``out`` has shape [N, M] (C^T row-major == C column-major with leading dimension M).
    """
    import torch
    _require_cuda_bf16(a, "a", 2)
    _require_cuda_bf16(b, "b", 2)
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((N, M), dtype=torch.bfloat16, device=a.device)
    torch.cuda.current_stream().synchronize()
    _check(library().b200_run_kernel(M, N, K, a.data_ptr(), b.data_ptr(), out.data_ptr(), None))
    torch.cuda.synchronize()
    return out


def reference_gpu_gemm(a, b, out=None, alpha: float = 1.0, beta: float = 0.0, stream=None):
    """The slow SIMT cross-check GEMM (reference.h:78-90 semantics), row-major C; bf16 or fp16."""
    import torch
    dtype = torch.float16 if a.dtype == torch.float16 else torch.bfloat16
    _require_cuda_bf16(a, "a", 2, dtype)
    _require_cuda_bf16(b, "b", 2, dtype)
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=dtype, device=a.device)
    fn = library().b200_reference_gpu_gemm_f16 if dtype == torch.float16 else library().b200_reference_gpu_gemm_bf16
    _check(fn(M, N, K, a.data_ptr(), b.data_ptr(), out.data_ptr(),
                                                  alpha, beta, _stream_ptr(stream)))
    return out


def gemm_host(a_bits, b_bits, out_bits=None, alpha: float = 1.0, beta: float = 0.0,
              cfg: Optional[GemmConfig] = None, copies_only: bool = False):
    """Host-buffer GEMM: numpy uint16 arrays holding bf16 bit patterns, [M,K] and [N,K].

    Copies to the device, multiplies and copies back inside the library (b200_gemm_bf16_host).
    Accepts torch CPU tensors (pinned or not) of dtype bfloat16 as well. ``copies_only`` runs the
    same host<->device copies without the kernels (b200_gemm_bf16_host_copies_only): the time the
    host links alone take, for benchmarks.
    """
    import numpy as np

    def ptr_shape(x):
        if isinstance(x, np.ndarray):
            if x.dtype != np.uint16 or not x.flags.c_contiguous:
                raise GemmError(STATUS_INVALID_ARG, "numpy operands must be C-contiguous uint16")
            return x.ctypes.data, x.shape
        return x.data_ptr(), tuple(x.shape)

    pa, (M, K) = ptr_shape(a_bits)
    pb, (N, Kb) = ptr_shape(b_bits)
    if K != Kb:
        raise GemmError(STATUS_INVALID_ARG, "a and b disagree on K")
    if out_bits is None:
        if isinstance(a_bits, np.ndarray):
            out_bits = np.empty((M, N), dtype=np.uint16)
        else:
            import torch
            out_bits = torch.empty((M, N), dtype=a_bits.dtype, pin_memory=a_bits.is_pinned())
    pc, _ = ptr_shape(out_bits)
    keep, p = _cfg_ptr(cfg)
    if copies_only:
        _check(library().b200_gemm_bf16_host_copies_only(M, N, K, pa, pb, pc))
    else:
        _check(library().b200_gemm_bf16_host(M, N, K, pa, pb, pc, alpha, beta, p))
    return out_bits


PROFILE_SLOTS = ("total", "producer_wait", "mma_wait_full", "mma_wait_tmem", "epi_wait_full", "epi_drain",
                 "epi_busy", "tiles")


def set_profile_buffer(buffer) -> None:
    """Registers (or, with None, removes) a CUDA int64 tensor of 8 counters per CTA that every
    launch fills with per-role cycle counts (see include/b200_gemm.h)."""
    if buffer is None:
        _check(library().b200_gemm_set_profile_buffer(None, 0))
    else:
        _check(library().b200_gemm_set_profile_buffer(buffer.data_ptr(), buffer.numel() * buffer.element_size()))


def selftest_bounded_wait(budget_cycles: int = 1 << 20) -> None:
    """Launches the kernel whose only wait is designed to run out (see include/b200_gemm.h)."""
    _check(library().b200_gemm_selftest_bounded_wait(budget_cycles))


def device_status():
    """Synchronises and returns (status_code, [role, block, tile, detail])."""
    words = (ctypes.c_uint * 4)()
    rc = library().b200_gemm_last_device_status(ctypes.byref(words))
    if rc not in (STATUS_OK, STATUS_DEVICE_TIMEOUT):
        _check(rc)
    return rc, list(words)
