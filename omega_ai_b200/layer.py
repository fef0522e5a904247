"""Host-side mirror of the engine's operator surface for the MoE layer.

The reference is a Java engine: a layer is built with ``(dims..., network)``,
driven with ``forward(Tensor)`` (``setInput; init(); output()``) and read with
``getOutput()`` (src/main/java/com/omega/engine/nn/layer/Layer.java:66-104;
LlamaMLPLayer.java:199-217).  No JDK exists in this build environment, so the
same surface is mirrored here in Python over the identical C ABI; the Java
sources that bind the ABI are under ``omega_ai_b200/java``.  torch is used only
to own device memory and streams.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import native
from .native import OMOE_BF16, OMOE_F32, Config, OmoeError, check


class Tensor:
    """4-D NCHW tensor with a host array and a device buffer, as
    src/main/java/com/omega/engine/tensor/Tensor.java:23-47.  ``data`` is the
    host ``float[]``; ``gpu`` is the device buffer (fp32 like the reference, or
    bf16 for the benchmark configurations)."""

    def __init__(self, number, channel, height, width, data=None, hasGPU=True, dtype=torch.float32,
                 device="cuda"):
        self.number, self.channel, self.height, self.width = number, channel, height, width
        self.dataLength = number * channel * height * width
        self.dtype = dtype
        if data is None:
            self.data = np.zeros(self.dataLength, np.float32)
        else:
            self.data = np.ascontiguousarray(data, np.float32).reshape(-1)
            assert self.data.size == self.dataLength
        self.gpu = None
        if hasGPU:
            self.gpu = torch.empty(self.dataLength, dtype=dtype, device=device)
            if data is not None:
                self.hostToDevice()

    @classmethod
    def from_device(cls, t: torch.Tensor):
        """Wrap an existing [N, W] device tensor without copying."""
        obj = cls.__new__(cls)
        obj.number, obj.channel, obj.height, obj.width = t.shape[0], 1, 1, t.shape[1]
        obj.dataLength = t.numel()
        obj.dtype = t.dtype
        obj.data = None
        obj.gpu = t.contiguous().view(-1)
        return obj

    def getGpuData(self) -> int:
        """Raw device address (what a JCuda Pointer wraps)."""
        return self.gpu.data_ptr()

    def hostToDevice(self):  # Tensor.java:571-579
        self.gpu.copy_(torch.from_numpy(self.data).to(self.dtype))
        torch.cuda.synchronize()

    def syncHost(self):  # Tensor.java:559-565
        self.data = self.gpu.float().cpu().numpy().reshape(-1)
        return self.data

    def view2d(self) -> torch.Tensor:
        return self.gpu.view(self.number, -1)


class Layer:
    """Subset of the abstract operator surface (Layer.java:66-104) this path uses."""

    def __init__(self, network=None):
        self.network = network
        self.input = None
        self.output_t = None
        self.number = 0

    def init(self):
        raise NotImplementedError

    def initParam(self):
        raise NotImplementedError

    def output(self):
        raise NotImplementedError

    def getOutput(self) -> Tensor:
        return self.output_t

    def setInput(self, input: Tensor):
        self.input = input

    def forward(self, input: Tensor) -> Tensor:  # LlamaMLPLayer.java:199-207
        self.setInput(input)
        self.init()
        self.output()
        return self.output_t


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return OMOE_F32
    if t == torch.bfloat16:
        return OMOE_BF16
    raise OmoeError(-1, f"unsupported dtype {t}")


class MoELayer(Layer):
    """Mixture-of-experts FFN that takes the slot of ``LlamaMLPLayer``
    (LlamaTransformerBlock.java:97,135).  Constructor arguments follow the Java
    layer: ``(embedDim, dff, numExperts, topK, bias, network)``.

    ``compute_dtype`` selects the arithmetic: ``torch.float32`` (the
    reference's precision) or ``torch.bfloat16`` (tensor cores, fp32
    accumulate).  ``t_max`` bounds the tokens of one forward.
    """

    def __init__(self, embedDim, dff, numExperts, topK, bias=False, network=None, *, t_max=4096,
                 compute_dtype=torch.bfloat16, renormalize=True, world=1, rank=0, recv_rows_max=0,
                 keep_weights=False):
        super().__init__(network)
        self.embedDim, self.dff, self.numExperts, self.topK = embedDim, dff, numExperts, topK
        self.hasBias = bool(bias)
        self.compute_dtype = compute_dtype
        self.t_max = t_max
        self.world, self.rank = world, rank
        self.keep_weights = keep_weights  # keep the source tensors so saveModel can write them
        self._h = C.c_void_p()
        cfg = Config(t_max=t_max, d_model=embedDim, d_ff=dff, n_experts=numExperts, top_k=topK,
                     compute_dtype=_dt(compute_dtype), renormalize=int(renormalize),
                     has_router_bias=int(self.hasBias), world=world, rank=rank, recv_rows_max=recv_rows_max)
        self._lib = native.lib()
        rc = self._lib.omoe_create(C.byref(cfg), C.byref(self._h))
        if rc != 0:
            raise OmoeError(rc, self._lib.omoe_last_error(None).decode())
        self._weights = None

    # ---- parameters ------------------------------------------------------
    def initParam(self, seed: int = 0, std: float = 0.02, device="cuda"):
        """Random N(0, std) weights, the convention of the benchmark configs
        (the reference initialises FullyLayer weights with RandomUtils.normal_,
        RandomUtils.java:697-703)."""
        g = torch.Generator(device=device).manual_seed(seed)
        E, El, d, dff = self.numExperts, self.numExperts // self.world, self.embedDim, self.dff
        dt = self.compute_dtype

        def rn(*shape):
            return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std).to(dt)

        w_router = rn(E, d)
        bias = rn(E) if self.hasBias else None
        self.setWeights(w_router, rn(El, dff, d), rn(El, dff, d), rn(El, d, dff), bias)

    def setWeights(self, w_router, w_gate, w_up, w_down, router_bias=None, stream=None):
        """All tensors on the device, same dtype, [out,in] row-major
        (FullyLayer.java:181): router [E,d]; gate/up [E_local,dff,d]
        (linear1/linear3); down [E_local,d,dff] (linear2)."""
        ts = [w_router, w_gate, w_up, w_down] + ([router_bias] if router_bias is not None else [])
        dt = w_router.dtype
        El = self.numExperts // self.world
        assert all(t.is_cuda and t.dtype == dt and t.is_contiguous() for t in ts)
        assert tuple(w_router.shape) == (self.numExperts, self.embedDim)
        assert tuple(w_gate.shape) == (El, self.dff, self.embedDim) == tuple(w_up.shape)
        assert tuple(w_down.shape) == (El, self.embedDim, self.dff)
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_set_weights(
            self._h, w_router.data_ptr(), router_bias.data_ptr() if router_bias is not None else None,
            w_gate.data_ptr(), w_up.data_ptr(), w_down.data_ptr(), _dt(dt), s))
        torch.cuda.current_stream().synchronize()
        self._weights = (w_router, w_gate, w_up, w_down, router_bias) if self.keep_weights else True

    # ---- checkpoint (the engine's headerless little-endian float32 stream) ----
    def saveModel(self, f):
        """Writes router (weight, bias), then per expert gate, up, down — the order
        LlamaMLPLayer.saveModel uses for linear1, linear3, linear2 (LlamaMLPLayer.java:273-277)."""
        from . import checkpoint

        if not isinstance(self._weights, tuple):
            raise OmoeError(-4, "saveModel needs the layer to be built with keep_weights=True")
        w_router, w_gate, w_up, w_down, bias = (None if t is None else t.float().cpu().numpy() for t in self._weights)
        checkpoint.write_moe(f, w_router, bias, w_gate, w_up, w_down)

    def loadModel(self, f, device="cuda"):
        from . import checkpoint

        El = self.numExperts // self.world
        assert self.world == 1, "load per rank: read the file and pass this rank's experts to setWeights"
        w_router, bias, w_gate, w_up, w_down = checkpoint.read_moe(f, self.numExperts, self.embedDim, self.dff, self.hasBias)
        dev = lambda a: None if a is None else torch.from_numpy(a).to(device).to(self.compute_dtype).contiguous()
        self.setWeights(dev(w_router), dev(w_gate[:El]), dev(w_up[:El]), dev(w_down[:El]), dev(bias))

    # ---- forward ---------------------------------------------------------
    def init(self):
        self.number = self.input.number
        if self.output_t is None or self.output_t.number != self.number or self.output_t.dtype != self.input.dtype:
            self.output_t = Tensor(self.number, 1, 1, self.embedDim, dtype=self.input.dtype,
                                   device=self.input.gpu.device)

    def output(self, stream=None):
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_forward(self._h, self.input.getGpuData(), self.output_t.getGpuData(),
                                              self.number, _dt(self.input.dtype), s))

    def forward_device(self, x: torch.Tensor, y: torch.Tensor | None = None, stream=None) -> torch.Tensor:
        """Raw-pointer call on [T, d] device tensors (no Tensor wrapper)."""
        assert x.is_cuda and x.is_contiguous() and x.shape[1] == self.embedDim
        if y is None:
            y = torch.empty_like(x)
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_forward(self._h, x.data_ptr(), y.data_ptr(), x.shape[0], _dt(x.dtype), s))
        return y

    def forward_block(self, x: torch.Tensor, gamma: torch.Tensor, y: torch.Tensor | None = None, eps: float = 1e-5,
                      stream=None) -> torch.Tensor:
        """y = x + MoE(rmsnorm(x) * gamma): norm2 -> mlp -> residual add of the transformer block
        (LlamaTransformerBlock.java:134-136) in one call. ``gamma`` [d] fp32 on the device."""
        assert x.is_cuda and x.is_contiguous() and gamma.is_cuda and gamma.dtype == torch.float32
        if y is None:
            y = torch.empty_like(x)
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_forward_block(self._h, x.data_ptr(), gamma.data_ptr(), eps, y.data_ptr(),
                                                    x.shape[0], _dt(x.dtype), s))
        return y

    # ---- training --------------------------------------------------------
    def set_training(self, on: bool = True):
        """Training mode: forwards keep what :meth:`backward` needs (the outputs of linear1, SiLU and
        linear3 that the reference's LlamaMLPLayer keeps, LlamaMLPLayer.java:117-123)."""
        check(self._h, self._lib.omoe_set_training(self._h, int(on)))

    def backward(self, x: torch.Tensor, dy: torch.Tensor, dx: torch.Tensor | None = None, stream=None) -> torch.Tensor:
        """LlamaMLPLayer.diff() for the MoE layer (LlamaMLPLayer.java:139-158): ``dy`` is the gradient of the
        last training-mode forward's output, ``x`` that forward's input; returns dx and leaves the weight
        gradients in the library (:meth:`weight_grads`)."""
        assert x.is_cuda and dy.is_cuda and x.is_contiguous() and dy.is_contiguous() and x.dtype == dy.dtype
        if dx is None:
            dx = torch.empty_like(x)
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_backward(self._h, x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.shape[0],
                                               _dt(x.dtype), s))
        return dx

    def backward_block(self, x: torch.Tensor, gamma: torch.Tensor, dy: torch.Tensor, eps: float = 1e-5, stream=None):
        """Backward of :meth:`forward_block`: returns (dx, dgamma); weight gradients via :meth:`weight_grads`."""
        assert x.is_cuda and dy.is_cuda and x.is_contiguous() and dy.is_contiguous() and x.dtype == dy.dtype
        dx = torch.empty_like(x)
        dgamma = torch.empty(self.embedDim, dtype=torch.float32, device=x.device)
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_backward_block(self._h, x.data_ptr(), gamma.data_ptr(), eps, dy.data_ptr(),
                                                     dx.data_ptr(), dgamma.data_ptr(), x.shape[0], _dt(x.dtype), s))
        return dx, dgamma

    def set_aux_loss(self, coef: float):
        """Weight of the auxiliary load-balancing loss E * sum_e f_e * P_e in the objective :meth:`backward` differentiates."""
        check(self._h, self._lib.omoe_set_aux_loss(self._h, float(coef)))

    def aux_loss(self) -> float:
        """The auxiliary load-balancing loss of the last forward."""
        v = C.c_float(0.0)
        check(self._h, self._lib.omoe_get_aux_loss(self._h, C.byref(v)))
        return float(v.value)

    def weight_grads(self, stream=None) -> dict:
        """fp32 device tensors d_router [E,d], d_bias [E], d_gate/d_up [El,dff,d], d_down [El,d,dff] of the last
        backward (diffW of the reference's FullyLayer, FullyLayer.java:292-301).  With expert parallelism El is
        this rank's share of the experts (their gradients are complete: all ranks' rows are here) and the
        router's gradients cover this rank's tokens only: sum them over the ranks."""
        E, d, dff = self.numExperts, self.embedDim, self.dff
        El = E // self.world
        mk = lambda *shape: torch.empty(*shape, dtype=torch.float32, device="cuda")
        g = dict(d_router=mk(E, d), d_bias=mk(E), d_gate=mk(El, dff, d), d_up=mk(El, dff, d), d_down=mk(El, d, dff))
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_get_weight_grads(self._h, g["d_router"].data_ptr(), g["d_bias"].data_ptr(),
                                                       g["d_gate"].data_ptr(), g["d_up"].data_ptr(),
                                                       g["d_down"].data_ptr(), s))
        return g

    def forward_host(self, x: torch.Tensor, y: torch.Tensor, stream=None) -> torch.Tensor:
        """Host buffers in and out (pinned for asynchronous copies): H2D, forward, D2H, sync."""
        assert not x.is_cuda and not y.is_cuda and x.is_contiguous() and y.is_contiguous()
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_forward_host(self._h, x.data_ptr(), y.data_ptr(), x.shape[0], _dt(x.dtype), s))
        return y

    def forward_host_async(self, x: torch.Tensor, y: torch.Tensor, stream=None) -> None:
        """:meth:`forward_host` without the final synchronise: enqueue, return; ``y`` is complete once
        :meth:`wait` has returned.  Calls made before the wait run in order with their copies overlapped."""
        assert not x.is_cuda and not y.is_cuda and x.is_contiguous() and y.is_contiguous()
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        check(self._h, self._lib.omoe_forward_host_async(self._h, x.data_ptr(), y.data_ptr(), x.shape[0],
                                                         _dt(x.dtype), s))

    def wait(self) -> None:
        """Host waits for everything enqueued on this layer and raises if a kernel reported a failure."""
        check(self._h, self._lib.omoe_wait(self._h))

    # ---- read-outs -------------------------------------------------------
    def routing(self, T: int):
        """(topk_idx [T,k], topk_w [T,k], counts [E], offsets [E+1], perm [T*k]) of the last forward."""
        k, E = self.topK, self.numExperts
        idx = np.empty((T, k), np.int32)
        w = np.empty((T, k), np.float32)
        counts = np.empty(E, np.int32)
        offsets = np.empty(E + 1, np.int32)
        perm = np.empty(T * k, np.int32)
        p = lambda a: a.ctypes.data_as(C.c_void_p)
        check(self._h, self._lib.omoe_get_routing(self._h, p(idx), p(w), p(counts), p(offsets), p(perm)))
        return idx, w, counts, offsets, perm

    def logits(self, T: int) -> np.ndarray:
        out = np.empty((T, self.numExperts), np.float32)
        check(self._h, self._lib.omoe_get_logits(self._h, out.ctypes.data_as(C.c_void_p)))
        return out

    def launch_count(self) -> int:
        return int(self._lib.omoe_last_launch_count(self._h))

    def set_profiling(self, on: bool):
        check(self._h, self._lib.omoe_set_profiling(self._h, int(on)))

    def stage_ms(self, back: int = 0) -> dict:
        """Device time of every stage of a profiled forward: the last one (``back`` = 0) or one of the 31 before
        it, so a run of forwards can be timed back to back and read afterwards."""
        ms = (C.c_float * native.N_STAGES)()
        check(self._h, self._lib.omoe_get_stage_ms_at(self._h, back, ms))
        return dict(zip(native.STAGE_NAMES, [float(v) for v in ms]))

    def ep_export(self) -> bytes:
        """This rank's IPC handles (control block, dispatch buffer, expert outputs)."""
        buf = C.create_string_buffer(native.EP_BLOB_BYTES)
        check(self._h, self._lib.omoe_ep_export(self._h, buf))
        return buf.raw

    def ep_import(self, blobs):
        """``blobs``: the exported handles of all ranks, in rank order."""
        assert len(blobs) == self.world and all(len(b) == native.EP_BLOB_BYTES for b in blobs)
        check(self._h, self._lib.omoe_ep_import(self._h, b"".join(blobs)))

    def ep_connect(self, group=None, store=None, timeout_s: float = 60.0, tag: str = "0"):
        """Exchange the handles and open the peers' buffers; returns once every rank has done so, after which
        forward may be called (collectively).

        Default: over torch.distributed (``all_gather_object`` + ``barrier`` on ``group``).  With ``store`` (any
        torch.distributed store, e.g. a ``TCPStore``) the exchange is a rendezvous with a deadline instead: every
        rank posts its blob under ``omoe_ep/<tag>/<rank>`` and waits at most ``timeout_s`` seconds for the
        others; a rank that never posts makes the others raise ``OmoeError(OMOE_ERR_COMM)`` naming it, rather
        than wait forever (the reference's CyclicBarrier, DP.java:74, does wait forever on a dead thread)."""
        import torch.distributed as dist

        if store is None:
            blobs = [None] * self.world
            dist.all_gather_object(blobs, self.ep_export(), group=group)
            self.ep_import(blobs)
            torch.cuda.synchronize()
            dist.barrier(group=group)
            return
        import datetime

        def rendezvous(phase, payload):
            store.set(f"omoe_ep/{tag}/{phase}/{self.rank}", payload)
            got = []
            for q in range(self.world):
                key = f"omoe_ep/{tag}/{phase}/{q}"
                try:
                    store.wait([key], datetime.timedelta(seconds=timeout_s))
                except Exception as e:  # the store raises its own error types on a deadline
                    raise OmoeError(-7, f"ep_connect: rank {q} did not post its {phase} within {timeout_s} s ({type(e).__name__})")
                got.append(store.get(key))
            return got

        blobs = rendezvous("handles", self.ep_export())
        self.ep_import([bytes(b) for b in blobs])
        torch.cuda.synchronize()
        rendezvous("opened", b"1")

    @staticmethod
    def ep_connect_local(layers):
        """All ranks in this process, one layer per GPU in rank order (the reference's threads-per-device mode,
        DP.java:68-94): peer access instead of IPC handles."""
        arr = (C.c_void_p * len(layers))(*[l._h for l in layers])
        rc = layers[0]._lib.omoe_ep_connect_local(arr, len(layers))
        for l in layers:
            if rc != 0 and l._lib.omoe_last_error(l._h):
                check(l._h, rc)
        if rc != 0:
            raise native.OmoeError(rc, "omoe_ep_connect_local")

    def close(self):
        if self._h:
            self._lib.omoe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
