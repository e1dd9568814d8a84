"""Projection stacks of a decoder, run through the quantized-linear path.

The timed path of the decode workloads is "the quantized projections, row-sharded": for a
7B-shape Llama layer that is Wq, Wk, Wv, Wo [4096 x 4096], Wgate, Wup [11008 x 4096] and
Wdown [4096 x 11008], 32 layers, every weight a distinct buffer in HBM.  Attention, norms
and activations lie outside this path, so each projection reads a fixed activation buffer
of its input width and the projections are issued in layer order on one stream; with more
than one rank every projection is followed by the all-gather of its row shards.  One step
(= one token) is recorded once as a CUDA graph and replayed.

Host-side orchestration only; all arithmetic happens in libwfb200 kernels.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from . import _native as N
from . import quant as Q
from .backend import CudaContext, QuantizedWeight


@dataclass(frozen=True)
class StackSpec:
    name: str
    qtype: Q.QuantizationType
    layers: int
    projections: tuple  # (name, rows, k)
    config: int         # benchmark config number, used for seeding

    def bytes_per_token(self) -> int:
        """Algorithmic weight bytes one token reads: GGUF block bytes of every projection."""
        return self.layers * sum(rows * self.qtype.row_bytes(k) for _, rows, k in self.projections)


LLAMA_7B_Q4_0 = StackSpec("7b-shape Q4_0", Q.QuantizationType.Q4_0, 32, (
    ("wq", 4096, 4096), ("wk", 4096, 4096), ("wv", 4096, 4096), ("wo", 4096, 4096),
    ("wgate", 11008, 4096), ("wup", 11008, 4096), ("wdown", 4096, 11008)), 4)

LLAMA_70B_Q4_K = StackSpec("70b-shape Q4_K", Q.QuantizationType.Q4_K, 80, (
    ("wq", 8192, 8192), ("wk", 1024, 8192), ("wv", 1024, 8192), ("wo", 8192, 8192),
    ("wgate", 28672, 8192), ("wup", 28672, 8192), ("wdown", 8192, 28672)), 5)


class Communicator:
    """NCCL communicator owned by the native library (wf_comm_*)."""

    def __init__(self, context: CudaContext, unique_id: bytes, rank: int, world: int):
        self.context, self.rank, self.world = context, rank, world
        h = ctypes.c_int64()
        buf = ctypes.create_string_buffer(unique_id, 128)
        context._ck("wf_comm_init", context._lib.wf_comm_init(context.handle, buf, rank, world, ctypes.byref(h)))
        self.handle = h.value

    @staticmethod
    def create_unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        N.check("wf_comm_get_unique_id", N.load().wf_comm_get_unique_id(buf))
        return buf.raw

    @property
    def peer_stores(self) -> bool:
        """True when small gathers of wf_qlinear_allgather go by stores into the peers' memory instead of NCCL."""
        flag = ctypes.c_int(0)
        c = self.context
        c._ck("wf_comm_info", c._lib.wf_comm_info(c.handle, self.handle, None, None, ctypes.byref(flag)))
        return bool(flag.value)

    def all_gather(self, send_dev: int, recv_dev: int, bytes_per_rank: int, stream: int = 0) -> None:
        c = self.context
        c._ck("wf_allgather", c._lib.wf_allgather(c.handle, self.handle, send_dev, recv_dev, bytes_per_rank, stream))

    def close(self) -> None:
        if self.handle and self.context.handle:
            h, self.handle = self.handle, 0
            self.context._ck("wf_comm_destroy", self.context._lib.wf_comm_destroy(self.context.handle, h))


class ProjectionStack:
    def __init__(self, context: CudaContext, spec: StackSpec, tokens: int = 1, comm: Optional[Communicator] = None,
                 layers: Optional[int] = None, rank: int = 0, world: int = 1):
        self.ctx, self.spec, self.m, self.comm = context, spec, tokens, comm
        self.rank = comm.rank if comm else rank
        self.world = comm.world if comm else world
        self.mode = "graph"  # "graph": one kernel (+ NCCL all-gather) per projection; "program": one persistent kernel
        self.layers = layers if layers is not None else spec.layers
        self.weights: List[List[QuantizedWeight]] = []
        self.blocks = {}
        self.x_host = {}
        self.x_dev = {}
        self.y_dev = {}
        self.graph = 0
        self._build()

    def _build(self) -> None:
        spec, ctx = self.spec, self.ctx
        for i, (name, rows, k) in enumerate(spec.projections):
            self.blocks[name] = Q.synth_weight(spec.qtype, rows, k, Q.config_seed(spec.config, i))
            if k not in self.x_host:
                self.x_host[k] = Q.synth_activation_bf16(self.m, k, Q.config_seed(spec.config, 100 + k))
                self.x_dev[k] = ctx.allocate(self.x_host[k].nbytes)
                ctx.copy_to_device(self.x_dev[k], self.x_host[k])
            self.y_dev[name] = ctx.allocate(self.m * rows * 4)
        for _ in range(self.layers):
            self.weights.append([QuantizedWeight(ctx, spec.qtype, self.blocks[name], rows, k, self.rank, self.world)
                                 for name, rows, k in spec.projections])

    def device_weight_bytes(self) -> int:
        return sum(w.device_bytes() for layer in self.weights for w in layer)

    def algorithmic_bytes_per_step(self) -> int:
        """GGUF block bytes this rank's shards hold, plus activations read and outputs written."""
        spec = self.spec
        per_layer = 0
        for name, rows, k in spec.projections:
            per_layer += (rows // self.world) * spec.qtype.row_bytes(k) + self.m * k * 2 + self.m * (rows // self.world) * 4
        return per_layer * self.layers

    def _issue(self, stream: int = 0) -> None:
        ctx, lib = self.ctx, self.ctx._lib
        for layer in self.weights:
            for w, (name, rows, k) in zip(layer, self.spec.projections):
                if self.comm is None:
                    rc = lib.wf_qlinear(ctx.handle, w.handle, self.x_dev[k], N.WF_DTYPE_BF16, 1, self.m,
                                        self.y_dev[name], 1, stream)
                    ctx._ck("wf_qlinear", rc)
                else:
                    rc = lib.wf_qlinear_allgather(ctx.handle, self.comm.handle, w.handle, self.x_dev[k], N.WF_DTYPE_BF16,
                                                  self.m, self.y_dev[name], stream)
                    ctx._ck("wf_qlinear_allgather", rc)

    # ---- the step as one persistent kernel ("program")
    OP_NEW_X, OP_DEPENDS = 1, 2

    def op_flags(self) -> List[int]:
        """Dependencies of a decoder layer: Wq/Wk/Wv read one input, Wo reads attention's output,
        Wgate/Wup read one input, Wdown reads the MLP product; each new input depends on what came
        before, so it needs every CTA (and rank) to have finished the previous projections."""
        new = self.OP_NEW_X | self.OP_DEPENDS
        starts_group = {"wq", "wo", "wgate", "wdown"}
        flags, prev_k = [], None
        for _ in range(self.layers):
            for name, _, k in self.spec.projections:
                # a projection that reads another buffer than its predecessor always stages anew
                flags.append(new if (name in starts_group or k != prev_k) else 0)
                prev_k = k
        return flags

    def export_buffers(self) -> dict:
        """IPC handles of this rank's landing buffers (one per output buffer), for the peers."""
        ctx, lib = self.ctx, self.ctx._lib
        if not hasattr(self, "landing_dev"):
            self.landing_dev = {}
            for name, rows, _ in self.spec.projections:
                nbytes = self.m * rows * 8
                self.landing_dev[name] = ctx.allocate(nbytes)
                ctx.copy_to_device(self.landing_dev[name], np.zeros(nbytes, np.uint8))
        out = {}
        for name, ptr in self.landing_dev.items():
            h = ctypes.create_string_buffer(64)
            ctx._ck("wf_ipc_export", lib.wf_ipc_export(ctx.handle, ptr, h))
            out[name] = h.raw
        return out

    def build_program(self, peer_handles: Optional[List[dict]] = None) -> None:
        """peer_handles[r] = export_buffers() of rank r (None for a single rank)."""
        ctx, lib = self.ctx, self.ctx._lib
        world, rank = self.world, self.rank
        self._imported = []
        landing_of = [dict() for _ in range(world)]
        if world > 1:
            landing_of[rank] = dict(self.landing_dev)
            for r in range(world):
                if r == rank:
                    continue
                for name, raw in peer_handles[r].items():
                    p = ctypes.c_int64()
                    ctx._ck("wf_ipc_import", lib.wf_ipc_import(ctx.handle, ctypes.create_string_buffer(raw, 64), ctypes.byref(p)))
                    self._imported.append(p.value)
                    landing_of[r][name] = p.value
        weights, xs, ys, lls = [], [], [], []
        for layer in self.weights:
            for w, (name, rows, k) in zip(layer, self.spec.projections):
                weights.append(w.handle)
                xs.append(self.x_dev[k])
                ys.append(self.y_dev[name])
                if world > 1:
                    lls.extend(landing_of[r][name] for r in range(world))
        n = len(weights)
        arr = lambda v, t: (t * len(v))(*v)
        prog = ctypes.c_int64()
        ctx._ck("wf_program_create", lib.wf_program_create(
            ctx.handle, n, arr(weights, ctypes.c_int64), arr(xs, ctypes.c_int64), arr(ys, ctypes.c_int64),
            arr(self.op_flags(), ctypes.c_int), self.m, world, rank,
            arr(lls, ctypes.c_int64) if world > 1 else None, ctypes.byref(prog)))
        self.program = prog.value

    def run_program(self, stream: int = 0) -> None:
        self.ctx._ck("wf_program_run", self.ctx._lib.wf_program_run(self.ctx.handle, self.program, stream))

    def record(self, stream: int = 0) -> None:
        """Issue one step eagerly (allocates whatever the kernels need), then record it."""
        self._issue(stream)
        self.ctx.synchronize(stream)
        self.ctx.graph_begin(stream)
        self._issue(stream)
        self.graph = self.ctx.graph_end(stream)

    def step(self, stream: int = 0) -> None:
        if self.mode == "program":
            self.run_program(stream)
        else:
            self.ctx.graph_launch(self.graph, stream)

    def step_host(self, x_host: dict, y_out: np.ndarray, pinned_in: dict, pinned_out: int, stream: int = 0) -> None:
        """One token end to end: this step's activations are written into pinned host memory, copied to the device,
        the step runs, the last projection's output comes back to pinned host memory, then wait."""
        ctx, lib = self.ctx, self.ctx._lib
        for k in self.x_dev:
            ctypes.memmove(pinned_in[k], x_host[k].ctypes.data, x_host[k].nbytes)
        last = self.spec.projections[-1][0]
        if self.mode == "program":  # copies, the kernel, the copy back and the wait in one native call
            if not hasattr(self, "_step_args"):
                ks = list(self.x_dev)
                self._step_args = ((ctypes.c_void_p * len(ks))(*[pinned_in[k] for k in ks]), (ctypes.c_int64 * len(ks))(*[self.x_dev[k] for k in ks]),
                                   (ctypes.c_int64 * len(ks))(*[x_host[k].nbytes for k in ks]), len(ks))
            src, dst, nb, n = self._step_args
            ctx._ck("wf_program_step_host", lib.wf_program_step_host(ctx.handle, self.program, n, src, dst, nb, pinned_out, self.y_dev[last],
                                                                      y_out.nbytes, stream))
        else:
            for k, dptr in self.x_dev.items():
                ctx._ck("wf_memcpy_h2d", lib.wf_memcpy_h2d(ctx.handle, dptr, pinned_in[k], x_host[k].nbytes, stream, 0))
            self.step(stream)
            ctx._ck("wf_memcpy_d2h", lib.wf_memcpy_d2h(ctx.handle, pinned_out, self.y_dev[last], y_out.nbytes, stream, 1))
        ctypes.memmove(y_out.ctypes.data, pinned_out, y_out.nbytes)

    def read_output(self, name: str) -> np.ndarray:
        rows = dict((n, r) for n, r, _ in self.spec.projections)[name]
        out = np.empty((self.m, rows), np.float32)
        self.ctx.copy_to_host(out, self.y_dev[name])
        return out

    def close(self) -> None:
        if getattr(self, "program", 0):
            self.ctx._ck("wf_program_destroy", self.ctx._lib.wf_program_destroy(self.ctx.handle, self.program))
            self.program = 0
        if self.graph:
            self.ctx.graph_destroy(self.graph)
            self.graph = 0
        for layer in self.weights:
            for w in layer:
                w.close()
        self.weights = []


class FusedDecoderStack:
    """A decoder's projections with the fp32 operations between them fused into the one-token program kernel
    (`wf_program_create_fused`): per layer

        q, k, v   = W{q,k,v} . rms_norm(h, gamma1)
        h_mid     = h + Wo . attn                       (attn: the attention block's output, supplied by the caller --
                                                         attention itself is outside this path)
        gate, up  = W{gate,up} . rms_norm(h_mid, gamma2)
        h_next    = h_mid + Wdown . (silu(gate) * up)

    All activations are fp32 device buffers that the projections read and write directly; one kernel launch per
    token.  Single rank.  `dims` = (d_model, ffn); weights are seeded synthetic blocks of `qtype`."""

    NAMES = ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown")

    def __init__(self, context: CudaContext, qtype: Q.QuantizationType, d_model: int, ffn: int, layers: int, seed: int = 11,
                 eps: float = 1e-5):
        self.ctx, self.qtype, self.d, self.ffn, self.layers, self.eps = context, qtype, d_model, ffn, layers, eps
        shapes = {"wq": (d_model, d_model), "wk": (d_model, d_model), "wv": (d_model, d_model), "wo": (d_model, d_model),
                  "wgate": (ffn, d_model), "wup": (ffn, d_model), "wdown": (d_model, ffn)}
        self.shapes = shapes
        rng = np.random.default_rng(seed)
        self.blocks, self.weights, self.gamma, self.host = [], [], [], {}
        self.dev = {}

        def buf(name, n, init=None):
            p = context.allocate(n * 4)
            a = np.zeros(n, np.float32) if init is None else np.ascontiguousarray(init, np.float32)
            context.copy_to_device(p, a)
            self.dev[name] = p
            self.host[name] = a
            return p

        buf("h0", d_model, rng.standard_normal(d_model))
        for l in range(layers):
            blk = {n: Q.synth_weight(qtype, r, k, seed * 1000 + l * 7 + i) for i, (n, (r, k)) in enumerate(shapes.items())}
            self.blocks.append(blk)
            self.weights.append({n: QuantizedWeight(context, qtype, blk[n], *shapes[n]) for n in self.NAMES})
            buf(f"gamma1_{l}", d_model, 1.0 + 0.1 * rng.standard_normal(d_model))
            buf(f"gamma2_{l}", d_model, 1.0 + 0.1 * rng.standard_normal(d_model))
            buf(f"attn_{l}", d_model, rng.standard_normal(d_model))
            for n in ("q", "k", "v", "hmid"):
                buf(f"{n}_{l}", d_model)
            buf(f"gate_{l}", ffn)
            buf(f"up_{l}", ffn)
            buf(f"h{l + 1}", d_model)
        self.program = 0
        self._build()

    def _build(self) -> None:
        ctx, lib, d = self.ctx, self.ctx._lib, self.dev
        new = ProjectionStack.OP_NEW_X | ProjectionStack.OP_DEPENDS
        W, X, Y, F, K, A, E, R = [], [], [], [], [], [], [], []

        def op(w, x, y, flags, kind=N.WF_X_BF16, aux=0, residual=0):
            W.append(w.handle); X.append(x); Y.append(y); F.append(flags); K.append(kind); A.append(aux); E.append(self.eps); R.append(residual)

        for l in range(self.layers):
            w = self.weights[l]
            op(w["wq"], d[f"h{l}"], d[f"q_{l}"], new, N.WF_X_RMSNORM_F32, d[f"gamma1_{l}"])
            op(w["wk"], d[f"h{l}"], d[f"k_{l}"], 0)
            op(w["wv"], d[f"h{l}"], d[f"v_{l}"], 0)
            op(w["wo"], d[f"attn_{l}"], d[f"hmid_{l}"], new, N.WF_X_F32, 0, d[f"h{l}"])
            op(w["wgate"], d[f"hmid_{l}"], d[f"gate_{l}"], new, N.WF_X_RMSNORM_F32, d[f"gamma2_{l}"])
            op(w["wup"], d[f"hmid_{l}"], d[f"up_{l}"], 0)
            op(w["wdown"], d[f"gate_{l}"], d[f"h{l + 1}"], new, N.WF_X_SWIGLU_F32, d[f"up_{l}"], d[f"hmid_{l}"])
        n = len(W)
        arr = lambda v, t: (t * len(v))(*v)
        prog = ctypes.c_int64()
        ctx._ck("wf_program_create_fused", lib.wf_program_create_fused(
            ctx.handle, n, arr(W, ctypes.c_int64), arr(X, ctypes.c_int64), arr(Y, ctypes.c_int64), arr(F, ctypes.c_int),
            arr(K, ctypes.c_int), arr(A, ctypes.c_int64), arr(E, ctypes.c_float), arr(R, ctypes.c_int64), 1, 1, 0, None,
            ctypes.byref(prog)))
        self.program = prog.value

    def weight_bytes_per_token(self) -> int:
        return self.layers * sum(r * self.qtype.row_bytes(k) for r, k in self.shapes.values())

    def run(self, stream: int = 0) -> None:
        self.ctx._ck("wf_program_run", self.ctx._lib.wf_program_run(self.ctx.handle, self.program, stream))

    def issue_unfused(self, stream: int = 0) -> None:
        """The same data flow as separate launches: every fp32 operation a kernel of its own (wf_rms_norm,
        wf_swiglu, wf_add) and every projection a wf_qlinear on one fp32 token -- twelve launches per layer.
        Needs scratch rows "x1", "x2", "act", "t" (allocated on first use)."""
        ctx, lib, d, h = self.ctx, self.ctx._lib, self.dev, self.ctx.handle
        if "x1" not in d:
            for n, size in (("x1", self.d), ("x2", self.d), ("act", self.ffn), ("t", self.d)):
                d[n] = ctx.allocate(size * 4)
                self.host[n] = np.zeros(size, np.float32)

        def lin(w, x, y):
            ctx._ck("wf_qlinear", lib.wf_qlinear(h, w.handle, x, N.WF_DTYPE_F32, 1, 1, y, 1, stream))

        for l in range(self.layers):
            w = self.weights[l]
            ctx._ck("wf_rms_norm", lib.wf_rms_norm(h, d[f"h{l}"], d[f"gamma1_{l}"], d["x1"], 1, self.d, self.eps, stream))
            lin(w["wq"], d["x1"], d[f"q_{l}"])
            lin(w["wk"], d["x1"], d[f"k_{l}"])
            lin(w["wv"], d["x1"], d[f"v_{l}"])
            lin(w["wo"], d[f"attn_{l}"], d["t"])
            ctx._ck("wf_add", lib.wf_add(h, d[f"h{l}"], d["t"], d[f"hmid_{l}"], self.d, stream))
            ctx._ck("wf_rms_norm", lib.wf_rms_norm(h, d[f"hmid_{l}"], d[f"gamma2_{l}"], d["x2"], 1, self.d, self.eps, stream))
            lin(w["wgate"], d["x2"], d[f"gate_{l}"])
            lin(w["wup"], d["x2"], d[f"up_{l}"])
            ctx._ck("wf_swiglu", lib.wf_swiglu(h, d[f"gate_{l}"], d[f"up_{l}"], d["act"], self.ffn, stream))
            lin(w["wdown"], d["act"], d["t"])
            ctx._ck("wf_add", lib.wf_add(h, d[f"hmid_{l}"], d["t"], d[f"h{l + 1}"], self.d, stream))

    def read(self, name: str) -> np.ndarray:
        out = np.empty_like(self.host[name])
        self.ctx.copy_to_host(out, self.dev[name])
        return out

    def close(self) -> None:
        if self.program:
            self.ctx._ck("wf_program_destroy", self.ctx._lib.wf_program_destroy(self.ctx.handle, self.program))
            self.program = 0
        for layer in self.weights:
            for w in layer.values():
                w.close()
        self.weights = []
        for p in self.dev.values():
            self.ctx.free(p)
        self.dev = {}
