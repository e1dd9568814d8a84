"""Host-side mirror of the reference's backend / kernel-operator API for the quantized
dot_general path, over the C ABI in include/wfb200.h.

The names follow the Java they stand in for (no JDK exists on the build or GPU machines,
so the host side is Python; a Java binding would wrap the same C entry points one to one):

* ``DotDimensionNumbers`` / ``DotGeneralOp`` -- the StableHLO records
  (snakeburger-core/src/main/java/io/surfworks/snakeburger/stablehlo/StableHloAst.java:211-239, 306-321).
* ``Tensor`` -- host tensor of shape + dtype + buffer
  (warpforge-core/src/main/java/io/surfworks/warpforge/core/tensor/Tensor.java:12-23).
* ``CudaContext`` -- allocate / free / copy / synchronize
  (warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/cuda/CudaContext.java:21-657).
* ``CudaOpKernel`` / ``QuantizedLinearKernel`` -- ``execute(op, inputs)``, ``supports(op)``,
  ``get_stream()`` (nvidia/ops/CudaOpKernel.java:12-36); the kernel validates like
  nvidia/ops/DotGeneralKernel.java:53-82, 169-226 and raises the same kinds of errors.
* ``NvidiaBackend`` -- ``name()``, ``execute``, ``supports``, ``close`` and the GpuBackend
  memory / stream calls (nvidia/NvidiaBackend.java:43-463;
  warpforge-core/.../core/backend/GpuBackend.java:12-154).  Unlike the reference, device
  memory and streams here are real, and there is no stub mode: construction fails without
  a B200.

A quantized weight crosses the boundary as ``QuantizedWeight``: an opaque, device-resident
handle with the logical shape [rows, k] of the rhs operand.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from . import _native as N
from .quant import QuantizationType


class UnsupportedOperationError(NotImplementedError):
    """java.lang.UnsupportedOperationException"""


class IllegalStateError(RuntimeError):
    """java.lang.IllegalStateException"""


@dataclass(frozen=True)
class DotDimensionNumbers:
    lhs_batching_dimensions: Sequence[int] = ()
    rhs_batching_dimensions: Sequence[int] = ()
    lhs_contracting_dimensions: Sequence[int] = (1,)
    rhs_contracting_dimensions: Sequence[int] = (0,)


@dataclass(frozen=True)
class DotGeneralOp:
    """``dimension_numbers`` may be None, as the reference allows (DotGeneralKernel.java:179)."""
    dimension_numbers: Optional[DotDimensionNumbers]
    result_shape: Sequence[int]
    result_dtype: str = "f32"


LINEAR_DIMS = DotDimensionNumbers((), (), (1,), (1,))  # torch.nn.functional.linear lowering


@dataclass
class Tensor:
    """Host tensor.  dtype 'f32' holds float32; 'bf16' holds the raw bits as uint16."""
    data: np.ndarray
    dtype: str = "f32"

    @staticmethod
    def from_float_array(values, *shape) -> "Tensor":
        a = np.asarray(values, np.float32)
        return Tensor(a.reshape(shape) if shape else a, "f32")

    @staticmethod
    def from_bf16_bits(bits, *shape) -> "Tensor":
        a = np.asarray(bits, np.uint16)
        return Tensor(a.reshape(shape) if shape else a, "bf16")

    def shape(self):
        return tuple(self.data.shape)

    def to_float_array(self) -> np.ndarray:
        if self.dtype == "bf16":
            return (self.data.astype(np.uint32) << 16).view(np.float32)
        return self.data.astype(np.float32)


@dataclass
class DeviceTensor:
    """Device-resident tensor: raw pointer + shape + dtype.  ``owner`` keeps whatever
    allocated the memory alive (a CudaContext allocation or, e.g., a torch tensor)."""
    ptr: int
    shape_: Sequence[int]
    dtype: str = "f32"
    owner: object = None

    def shape(self):
        return tuple(self.shape_)

    def nbytes(self) -> int:
        return int(np.prod(self.shape_)) * (4 if self.dtype == "f32" else 2)


class CudaContext:
    def __init__(self, device_index: int = 0):
        self._lib = N.load()
        h = ctypes.c_int64(0)
        N.check("wf_init", self._lib.wf_init(device_index, ctypes.byref(h)))
        self.handle = h.value
        self.device_index = device_index

    @staticmethod
    def device_count() -> int:
        n = ctypes.c_int(0)
        rc = N.load().wf_device_count(ctypes.byref(n))
        return n.value if rc == N.WF_OK else 0

    def _ck(self, op, rc):
        N.check(op, rc, self.handle)

    def device_info(self) -> dict:
        sm, ma, mi = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        tot, free = ctypes.c_int64(), ctypes.c_int64()
        self._ck("wf_device_info", self._lib.wf_device_info(self.handle, sm, ma, mi, tot, free))
        return {"sm_count": sm.value, "cc": (ma.value, mi.value), "total_mem": tot.value, "free_mem": free.value}

    def allocate(self, nbytes: int) -> int:
        p = ctypes.c_int64()
        self._ck("wf_malloc", self._lib.wf_malloc(self.handle, nbytes, ctypes.byref(p)))
        return p.value

    def free(self, dptr: int) -> None:
        self._ck("wf_free", self._lib.wf_free(self.handle, dptr))

    def host_alloc(self, nbytes: int) -> int:
        """Pinned host memory (GpuBackend.allocatePinned)."""
        p = ctypes.c_void_p()
        self._ck("wf_host_alloc", self._lib.wf_host_alloc(self.handle, nbytes, ctypes.byref(p)))
        return p.value

    def host_free(self, ptr: int) -> None:
        self._ck("wf_host_free", self._lib.wf_host_free(self.handle, ptr))

    def set_salt(self, salt: int) -> None:
        self._ck("wf_set_salt", self._lib.wf_set_salt(self.handle, salt))

    def copy_to_device(self, dptr: int, host: np.ndarray, stream: int = 0, sync: bool = True) -> None:
        host = np.ascontiguousarray(host)
        self._ck("wf_memcpy_h2d", self._lib.wf_memcpy_h2d(self.handle, dptr, host.ctypes.data, host.nbytes, stream, int(sync)))

    def copy_to_host(self, host: np.ndarray, dptr: int, stream: int = 0, sync: bool = True) -> None:
        assert host.flags.c_contiguous
        self._ck("wf_memcpy_d2h", self._lib.wf_memcpy_d2h(self.handle, host.ctypes.data, dptr, host.nbytes, stream, int(sync)))

    def set_exact_exp(self, on: bool) -> None:
        """silu / swiglu / softmax with the exponential evaluated as (float) Math.exp(x) (slower, bit-exact)."""
        self._ck("wf_set_exact_exp", self._lib.wf_set_exact_exp(self.handle, int(on)))

    def create_stream(self) -> int:
        s = ctypes.c_int64()
        self._ck("wf_stream_create", self._lib.wf_stream_create(self.handle, ctypes.byref(s)))
        return s.value

    def destroy_stream(self, stream: int) -> None:
        self._ck("wf_stream_destroy", self._lib.wf_stream_destroy(self.handle, stream))

    def synchronize(self, stream: int = 0) -> None:
        self._ck("wf_stream_sync", self._lib.wf_stream_sync(self.handle, stream))

    def create_event(self) -> int:
        e = ctypes.c_int64()
        self._ck("wf_event_create", self._lib.wf_event_create(self.handle, ctypes.byref(e)))
        return e.value

    def record_event(self, event: int, stream: int = 0) -> None:
        self._ck("wf_event_record", self._lib.wf_event_record(self.handle, event, stream))

    def elapsed_ms(self, start: int, stop: int) -> float:
        ms = ctypes.c_float()
        self._ck("wf_event_elapsed_ms", self._lib.wf_event_elapsed_ms(self.handle, start, stop, ctypes.byref(ms)))
        return ms.value

    def graph_begin(self, stream: int = 0) -> None:
        self._ck("wf_graph_begin", self._lib.wf_graph_begin(self.handle, stream))

    def graph_end(self, stream: int = 0) -> int:
        g = ctypes.c_int64()
        self._ck("wf_graph_end", self._lib.wf_graph_end(self.handle, stream, ctypes.byref(g)))
        return g.value

    def graph_launch(self, graph: int, stream: int = 0) -> None:
        self._ck("wf_graph_launch", self._lib.wf_graph_launch(self.handle, graph, stream))

    def graph_destroy(self, graph: int) -> None:
        self._ck("wf_graph_destroy", self._lib.wf_graph_destroy(self.handle, graph))

    def launch_count(self) -> int:
        n = ctypes.c_int64()
        self._ck("wf_launch_count", self._lib.wf_launch_count(self.handle, ctypes.byref(n)))
        return n.value

    def close(self) -> None:
        if self.handle:
            h, self.handle = self.handle, 0
            N.check("wf_destroy", self._lib.wf_destroy(h))


class QuantizedWeight:
    """Device-resident GGUF-quantized rhs operand of logical shape [rows, k]."""

    def __init__(self, context: CudaContext, qtype: QuantizationType, blocks: np.ndarray, rows: int, k: int,
                 shard_rank: int = 0, shard_world: int = 1):
        self.context, self.qtype = context, qtype
        blocks = np.ascontiguousarray(blocks, np.uint8)
        expect = rows * (k // qtype.block_size()) * qtype.bytes_per_block() if k % qtype.block_size() == 0 else -1
        if expect >= 0 and blocks.size != expect:
            raise ValueError(f"{qtype.name} tensor [{rows} x {k}] needs {expect} bytes, got {blocks.size}")
        h = ctypes.c_int64()
        context._ck("wf_weight_upload", context._lib.wf_weight_upload(
            context.handle, qtype.ggml_type, blocks.ctypes.data, rows, k, shard_rank, shard_world, ctypes.byref(h)))
        self.handle = h.value
        self.total_rows, self.k = rows, k
        self.rows = rows // shard_world
        self.row0 = self.rows * shard_rank
        self.shard_rank, self.shard_world = shard_rank, shard_world

    @classmethod
    def from_gguf(cls, context: "CudaContext", gguf_file, name: str, shard_rank: int = 0, shard_world: int = 1,
                  q4_0_order: int = N.WF_Q4_0_ORDER_REFERENCE) -> "QuantizedWeight":
        """Upload the 2-D tensor `name` of an open GGUF file ({k, rows} in file order) straight
        from the library's mapping of the file (wf_gguf_upload)."""
        info = gguf_file.tensor_info(name)
        h = ctypes.c_int64()
        context._ck("wf_gguf_upload", context._lib.wf_gguf_upload(
            context.handle, gguf_file.handle, name.encode(), shard_rank, shard_world, q4_0_order, ctypes.byref(h)))
        self = cls.__new__(cls)
        self.context, self.qtype = context, QuantizationType.from_ggml(info.ggml_type)
        self.handle = h.value
        self.k, self.total_rows = info.shape[0], info.shape[1]
        self.rows = self.total_rows // shard_world
        self.row0 = self.rows * shard_rank
        self.shard_rank, self.shard_world = shard_rank, shard_world
        return self

    def shape(self):
        return (self.rows, self.k)

    def device_bytes(self) -> int:
        b = ctypes.c_int64()
        self.context._ck("wf_weight_info", self.context._lib.wf_weight_info(
            self.context.handle, self.handle, None, None, None, None, ctypes.byref(b)))
        return b.value

    def dequantize_to_array(self, row0: int = 0, nrows: Optional[int] = None) -> np.ndarray:
        """QuantizedTensorView.dequantizeToArray (QuantizedTensorView.java:161-166), run on the device."""
        nrows = self.rows - row0 if nrows is None else nrows
        out = np.empty((max(nrows, 0), self.k), np.float32)
        self.context._ck("wf_dequant_rows", self.context._lib.wf_dequant_rows(
            self.context.handle, self.handle, row0, nrows, out.ctypes.data))
        return out

    def close(self) -> None:
        if self.handle and self.context.handle:
            h, self.handle = self.handle, 0
            self.context._ck("wf_weight_free", self.context._lib.wf_weight_free(self.context.handle, h))


class CudaOpKernel:
    def execute(self, op, inputs: List) -> List:
        raise NotImplementedError

    def supports(self, op) -> bool:
        return True

    def get_stream(self) -> int:
        return 0


class QuantizedLinearKernel(CudaOpKernel):
    """dot_general whose rhs is a QuantizedWeight: lhs [M, K] (contract 1) x rhs [N, K]
    (contract 1) -> [M, N] fp32.  Constructed (context, salt) like every reference kernel."""

    def __init__(self, context: CudaContext, salt: int = 0, stream: int = 0):
        self.context, self.salt, self.stream = context, salt, stream

    def get_stream(self) -> int:
        return self.stream

    def supports(self, op) -> bool:
        return isinstance(op, DotGeneralOp)

    def execute(self, op, inputs: List) -> List:
        if not isinstance(op, DotGeneralOp):
            raise ValueError(f"Expected DotGeneralOp, got: {type(op).__name__}")
        if len(inputs) != 2:
            raise ValueError(f"DotGeneral requires 2 inputs (lhs, rhs), got: {len(inputs)}")
        lhs, rhs = inputs
        if not isinstance(rhs, QuantizedWeight):
            raise UnsupportedOperationError("rhs is not a quantized weight; the fp32 dot_general path is not part of this library")
        lhs_shape = tuple(lhs.shape())
        if len(lhs_shape) != 2:
            raise UnsupportedOperationError(
                f"Only 2D and 3D (batched) matmul are currently supported. Got lhs dim={len(lhs_shape)}, rhs dim=2")
        lc, rc = 1, 0
        dn = op.dimension_numbers
        if dn is not None:
            if len(dn.lhs_contracting_dimensions) != 1 or len(dn.rhs_contracting_dimensions) != 1:
                raise UnsupportedOperationError("Only single contracting dimension supported for 2D matmul")
            if len(dn.lhs_batching_dimensions) or len(dn.rhs_batching_dimensions):
                raise UnsupportedOperationError("Batching dimensions are not supported for a quantized rhs")
            lc, rc = int(dn.lhs_contracting_dimensions[0]), int(dn.rhs_contracting_dimensions[0])
        if lc != 1 or rc != 1:
            raise UnsupportedOperationError(
                "A quantized rhs is stored [N, K] with blocks along K: only lhs_contract=[1], rhs_contract=[1] (linear) is supported")
        m, k = lhs_shape
        n, k2 = rhs.shape()
        if k != k2:
            raise ValueError(f"Contracting dimensions must match: K={k} vs K2={k2} (transposeA=False, transposeB=True)")
        if tuple(op.result_shape) != (m, n):
            raise ValueError(f"Result type {tuple(op.result_shape)} does not match [{m}, {n}]")
        dt = {"f32": N.WF_DTYPE_F32, "bf16": N.WF_DTYPE_BF16}.get(lhs.dtype)
        if dt is None:
            raise UnsupportedOperationError(f"lhs dtype {lhs.dtype} not supported")
        lib, ctx = self.context._lib, self.context
        if isinstance(lhs, DeviceTensor):
            out = DeviceTensor(ctx.allocate(m * n * 4), (m, n), "f32", owner=ctx)
            ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, rhs.handle, lhs.ptr, dt, 1, m, out.ptr, 1, self.stream))
            return [out]
        x = np.ascontiguousarray(lhs.data)
        y = np.empty((m, n), np.float32)
        ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, rhs.handle, x.ctypes.data, dt, 0, m, y.ctypes.data, 0, self.stream))
        return [Tensor(y, "f32")]


@dataclass(frozen=True)
class CustomCallOp:
    """stablehlo.custom_call: only the target name and the result shape matter to the kernels
    (the reference's CustomCallOp carries no parsed attributes either, CustomCallKernel.java:414-419)."""
    call_target: str
    result_shape: Sequence[int]
    result_dtype: str = "f32"


@dataclass(frozen=True)
class AddOp:
    """stablehlo.add on two fp32 tensors of one shape (the residual connection)."""
    result_shape: Sequence[int]


@dataclass(frozen=True)
class DotOp:
    """stablehlo.dot: [M,K] x [K,N], [M,K] x [K], [K] x [K,N] or [K] x [K] on dense fp32 tensors
    (snakeburger-core/.../stablehlo/StableHloAst.java DotOp)."""
    result_shape: Sequence[int]


@dataclass(frozen=True)
class MultiplyOp:
    """stablehlo.multiply; only the fused form silu(gate) * up exists on the device (``swiglu``)."""
    result_shape: Sequence[int]


DEFAULT_EPS = 1e-5  # CustomCallKernel.java:421


class CudaCustomCallKernel(CudaOpKernel):
    """Mirror of nvidia/ops/CudaCustomCallKernel.java:30-66: dispatch on the call target; host tensors
    are copied to the device, the kernel runs, the result comes back (as the reference does per call);
    DeviceTensor inputs stay on the device and the call only enqueues.  Targets: rms_norm, layer_norm,
    softmax, silu, embedding, plus ``swiglu`` (silu(gate) * up in one pass)."""

    TARGETS = ("rms_norm", "layer_norm", "softmax", "silu", "gelu", "embedding", "swiglu")

    def __init__(self, context: CudaContext, salt: int = 0, stream: int = 0):
        self.context, self.salt, self.stream = context, salt, stream

    def get_stream(self) -> int:
        return self.stream

    def supports(self, op) -> bool:
        return isinstance(op, (CustomCallOp, AddOp))

    def _to_device(self, t, temps, dtype=np.float32):
        if isinstance(t, DeviceTensor):
            return t.ptr
        a = np.ascontiguousarray(t.data if isinstance(t, Tensor) else t, dtype)
        p = self.context.allocate(max(a.nbytes, 4))
        temps.append(p)
        if a.nbytes:
            self.context.copy_to_device(p, a, self.stream, sync=True)
        return p

    def execute(self, op, inputs: List) -> List:
        ctx, lib, s = self.context, self.context._lib, self.stream
        target = "add" if isinstance(op, AddOp) else op.call_target
        if target not in self.TARGETS + ("add",):
            raise UnsupportedOperationError(f"Unknown custom_call target for CUDA: {target}")
        on_device = isinstance(inputs[0], DeviceTensor)
        temps: List[int] = []
        try:
            shape = tuple(inputs[0].shape())
            if target == "embedding":
                table_shape = tuple(inputs[1].shape())
                out_shape = shape + (table_shape[1],)
                count = int(np.prod(shape)) if shape else 1
                idx = self._to_device(inputs[0], temps, np.int64)
                table = self._to_device(inputs[1], temps)
                out = ctx.allocate(max(count * table_shape[1] * 4, 4))
                ctx._ck("wf_embedding", lib.wf_embedding(ctx.handle, idx, table, out, count, table_shape[0], table_shape[1], s))
            else:
                out_shape = shape
                n = shape[-1] if shape else 1
                total = int(np.prod(shape)) if shape else 1
                rows = total // n if n else 0
                ptrs = [self._to_device(t, temps) for t in inputs]
                out = ctx.allocate(max(total * 4, 4))
                opt = lambda i: ptrs[i] if len(ptrs) > i else 0
                if target == "rms_norm":
                    rc = lib.wf_rms_norm(ctx.handle, ptrs[0], opt(1), out, rows, n, DEFAULT_EPS, s)
                elif target == "layer_norm":
                    rc = lib.wf_layer_norm(ctx.handle, ptrs[0], opt(1), opt(2), out, rows, n, DEFAULT_EPS, s)
                elif target == "softmax":
                    rc = lib.wf_softmax(ctx.handle, ptrs[0], out, rows, n, s)
                elif target == "silu":
                    rc = lib.wf_silu(ctx.handle, ptrs[0], out, total, s)
                elif target == "gelu":
                    rc = lib.wf_gelu(ctx.handle, ptrs[0], out, total, s)
                else:
                    if len(ptrs) != 2 or tuple(inputs[1].shape()) != shape:
                        raise ValueError(f"{target} requires 2 inputs of one shape")
                    fn = lib.wf_swiglu if target == "swiglu" else lib.wf_add
                    rc = fn(ctx.handle, ptrs[0], ptrs[1], out, total, s)
                ctx._ck("wf_" + target, rc)
            if on_device:
                return [DeviceTensor(out, out_shape, "f32", owner=ctx)]
            host = np.empty(out_shape, np.float32)
            try:
                if host.nbytes:
                    ctx.copy_to_host(host, out, s, sync=True)
                ctx.synchronize(s)  # reports an embedding index outside the table
            finally:
                ctx.free(out)
            return [Tensor(host, "f32")]
        finally:
            for p in temps:  # wf_free waits for the device, so work that still reads them has finished
                ctx.free(p)


class DotKernel(CudaOpKernel):
    """Mirror of nvidia/ops/DotKernel.java:18-154 (C[M,N] = A[M,K] * B[K,N], fp32), with the vector forms of the CPU
    kernel (cpu/ops/scalar/DotKernel.java:18-102: [K] x [K] -> [1], [M,K] x [K] -> [M], [K] x [K,N] -> [N]).  Host tensors
    are copied to the device, the kernel runs, the result comes back; DeviceTensor inputs stay on the device."""

    def __init__(self, context: CudaContext, salt: int = 0, stream: int = 0):
        self.context, self.salt, self.stream = context, salt, stream

    def supports(self, op) -> bool:
        return isinstance(op, DotOp)

    def execute(self, op, inputs: List) -> List:
        if not isinstance(op, DotOp):
            raise ValueError(f"Expected DotOp, got: {type(op).__name__}")
        if len(inputs) != 2:
            raise ValueError(f"Dot requires exactly 2 inputs, got: {len(inputs)}")
        lhs, rhs = inputs
        ls, rs = tuple(lhs.shape()), tuple(rhs.shape())
        if len(ls) == 1 and len(rs) == 1:
            m, k, k2, n, out_shape = 1, ls[0], rs[0], 1, (1,)
        elif len(ls) == 2 and len(rs) == 2:
            m, k, k2, n, out_shape = ls[0], ls[1], rs[0], rs[1], (ls[0], rs[1])
        elif len(ls) == 2 and len(rs) == 1:
            m, k, k2, n, out_shape = ls[0], ls[1], rs[0], 1, (ls[0],)
        elif len(ls) == 1 and len(rs) == 2:
            m, k, k2, n, out_shape = 1, ls[0], rs[0], rs[1], (rs[1],)
        else:
            raise UnsupportedOperationError(f"Dot operation not supported for shapes: {list(ls)} x {list(rs)}")
        if k != k2:
            raise ValueError(f"Inner dimensions must match: A[{m},{k}] * B[{k2},{n}]")
        for t in (lhs, rhs):
            if t.dtype != "f32":
                raise ValueError("Dot requires fp32 tensors")
        ctx, lib, s = self.context, self.context._lib, self.stream
        on_device = all(isinstance(t, DeviceTensor) for t in inputs)
        temps, ptrs = [], []
        try:
            for t in inputs:
                if isinstance(t, DeviceTensor):
                    ptrs.append(t.ptr)
                else:
                    a = np.ascontiguousarray(t.data, np.float32)
                    p = ctx.allocate(max(a.nbytes, 4))
                    temps.append(p)
                    if a.nbytes:
                        ctx.copy_to_device(p, a, s)
                    ptrs.append(p)
            out = ctx.allocate(max(m * n * 4, 4))
            ctx._ck("wf_dot_f32", lib.wf_dot_f32(ctx.handle, ptrs[0], ptrs[1], out, m, n, k, s))
            if on_device:
                return [DeviceTensor(out, out_shape, "f32", owner=ctx)]
            host = np.empty(out_shape, np.float32)
            try:
                if host.nbytes:
                    ctx.copy_to_host(host, out, s, sync=True)
            finally:
                ctx.free(out)
            return [Tensor(host, "f32")]
        finally:
            for p in temps:
                ctx.free(p)


class NvidiaBackend:
    def __init__(self, device_index: int = 0, salt: int = 0):
        self._device_index, self._salt = device_index, salt
        self.cuda_context = CudaContext(device_index)
        glue = CudaCustomCallKernel(self.cuda_context, salt)
        self._kernels = {DotGeneralOp: QuantizedLinearKernel(self.cuda_context, salt), CustomCallOp: glue, AddOp: glue,
                         DotOp: DotKernel(self.cuda_context, salt)}
        self._closed = False
        self._weights: List[QuantizedWeight] = []

    def name(self) -> str:
        return "nvidia"

    def device_index(self) -> int:
        return self._device_index

    def _check_not_closed(self):
        if self._closed:
            raise IllegalStateError("Backend has been closed")

    def supports(self, op) -> bool:
        k = self._kernels.get(type(op))
        return k is not None and k.supports(op)

    def execute(self, op, inputs: List) -> List:
        self._check_not_closed()
        k = self._kernels.get(type(op))
        if k is None:
            raise UnsupportedOperationError(f"Operation not supported: {type(op).__name__}")
        return k.execute(op, list(inputs))

    def upload_weight(self, qtype: QuantizationType, blocks, rows: int, k: int, shard_rank: int = 0,
                      shard_world: int = 1) -> QuantizedWeight:
        self._check_not_closed()
        w = QuantizedWeight(self.cuda_context, qtype, blocks, rows, k, shard_rank, shard_world)
        self._weights.append(w)
        return w

    def upload_gguf_weight(self, gguf_file, name: str, shard_rank: int = 0, shard_world: int = 1,
                           q4_0_order: int = N.WF_Q4_0_ORDER_REFERENCE) -> QuantizedWeight:
        """Linear weight `name` of an open warpforge_b200.gguf.GGUF file, from the file mapping to the device."""
        self._check_not_closed()
        w = QuantizedWeight.from_gguf(self.cuda_context, gguf_file, name, shard_rank, shard_world, q4_0_order)
        self._weights.append(w)
        return w

    # --- GpuBackend memory / stream surface
    def allocate_device(self, shape, dtype: str = "f32") -> DeviceTensor:
        self._check_not_closed()
        nbytes = int(np.prod(shape)) * (4 if dtype == "f32" else 2)
        return DeviceTensor(self.cuda_context.allocate(nbytes), tuple(shape), dtype, owner=self.cuda_context)

    def copy_to_device(self, host: Tensor, stream: int = 0) -> DeviceTensor:
        self._check_not_closed()
        d = self.allocate_device(host.shape(), host.dtype)
        self.cuda_context.copy_to_device(d.ptr, host.data, stream)
        return d

    def copy_to_host(self, dev: DeviceTensor, stream: int = 0) -> Tensor:
        self._check_not_closed()
        a = np.empty(dev.shape(), np.float32 if dev.dtype == "f32" else np.uint16)
        self.cuda_context.copy_to_host(a, dev.ptr, stream)
        return Tensor(a, dev.dtype)

    def create_stream(self) -> int:
        self._check_not_closed()
        return self.cuda_context.create_stream()

    def destroy_stream(self, stream: int) -> None:
        self._check_not_closed()
        self.cuda_context.destroy_stream(stream)

    def synchronize_stream(self, stream: int = 0) -> None:
        self._check_not_closed()
        self.cuda_context.synchronize(stream)

    def synchronize_device(self) -> None:
        self.synchronize_stream(0)

    def total_device_memory(self) -> int:
        return self.cuda_context.device_info()["total_mem"]

    def free_device_memory(self) -> int:
        return self.cuda_context.device_info()["free_mem"]

    def used_device_memory(self) -> int:
        i = self.cuda_context.device_info()
        return i["total_mem"] - i["free_mem"]

    def close(self) -> None:
        if not self._closed:  # double close is safe (NvidiaBackendTest.java:185-199)
            self._closed = True
            self.cuda_context.close()
