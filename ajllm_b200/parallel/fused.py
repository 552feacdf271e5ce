"""Tensor-parallel projections fused with their collective over symmetric NVLink memory.

``gather_linear`` (column-parallel, all-gather -> GEMM) and ``linear_scatter`` (row-parallel, GEMM ->
reduce-scatter) each run as one persistent tcgen05 kernel per rank (``csrc/comm_gemm.cu``): remote
activation shards are pulled from the peers' symmetric staging buffers by copy CTAs while the compute
CTAs already work on the local shard, and partial output tiles are stored by the epilogue directly
into the owning rank's symmetric receive buffer. The backward passes are the mirrored kernels
(all-gather <-> reduce-scatter) plus a local weight-gradient GEMM. Symmetric buffers and flag words
come from ``torch.distributed._symmetric_memory``; the NCCL path in
:mod:`ajllm_b200.parallel.tensor_parallel` is the baseline these kernels are measured against.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ajllm_b200.ops import native
from ajllm_b200.ops.functional import gemm, wgrad_accumulate
from ajllm_b200.utils.timing import nvtx_range

_MAX_RANKS = 8
MODE_ALL_GATHER, MODE_REDUCE_SCATTER, MODE_ALL_REDUCE, MODE_GATHER_WEIGHT = 0, 1, 2, 3


class _CommArgs(ctypes.Structure):
    _fields_ = [
        ("mode", ctypes.c_int), ("m", ctypes.c_int), ("n", ctypes.c_int), ("k", ctypes.c_int),
        ("tp", ctypes.c_int), ("rank", ctypes.c_int), ("b_mn_major", ctypes.c_int), ("copy_ctas", ctypes.c_int),
        ("ldb", ctypes.c_longlong), ("ldc", ctypes.c_longlong),
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("out", ctypes.c_void_p), ("gathered", ctypes.c_void_p),
        ("stage_ptrs", ctypes.c_void_p * _MAX_RANKS), ("recv_ptrs", ctypes.c_void_p * _MAX_RANKS),
        ("recv_ptrs_even", ctypes.c_void_p * _MAX_RANKS),
        ("counter_ptrs", ctypes.c_void_p * _MAX_RANKS), ("ready_ptrs", ctypes.c_void_p * _MAX_RANKS),
        ("done_ptrs", ctypes.c_void_p * _MAX_RANKS),
        ("shard_flags", ctypes.c_void_p), ("reduce_state", ctypes.c_void_p), ("epoch", ctypes.c_uint),
        ("a_rows", ctypes.c_int), ("shard_elems", ctypes.c_longlong), ("b_offset_elems", ctypes.c_longlong),
        ("swiglu", ctypes.c_int), ("aux", ctypes.c_void_p), ("ld_aux", ctypes.c_longlong),
    ]


class FusedTensorParallel:
    BLOCK_M, BLOCK_N = 128, 256
    GUARD_BYTES, GUARD_PATTERN = 4096, 0xA5

    def __init__(self, group, device: torch.device, copy_ctas: int | None = None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.group = group
        self.device = device
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 2 <= self.size <= _MAX_RANKS:
            raise ValueError("fused tensor parallelism supports 2..8 ranks")
        # CTAs that pull the peers' shards before they join the products. Two ranks hide their one transfer behind the
        # products with 20; from four ranks on the transfer is the longer part and more pulling SMs shorten it
        # (measured on four GPUs: 588 / 485 / 472 / 444 us for the QKV gather with 20 / 32 / 48 / 64)
        fixed = copy_ctas or os.environ.get("AJB_COPY_CTAS")
        self.copy_ctas = int(fixed or ("20" if self.size <= 2 else "48"))
        # pulling CTAs of a gather whose transfer outlasts its products (`AJB_COPY_CTAS_LINK`). Same count by default:
        # on eight ranks 96 instead of 48 moved no more bytes per second (377 against 429 GB/s) and kept the SMs from the
        # products, 1418 against 918 us for the W13 gather
        self.copy_ctas_link_bound = int(fixed or os.environ.get("AJB_COPY_CTAS_LINK", str(self.copy_ctas)))
        # Buffers that peers read (staging) or write (receive) exist twice and alternate with the call number, so a
        # call never waits for its peers to finish the same call (csrc/comm_gemm.cu explains the protocol). Gathering
        # calls are counted here; reducing calls are counted on the device so that CUDA graphs can replay them.
        self.gather_calls = 0
        self._retired: list = []
        self._stage = [None, None]
        self._recv = [None, None]
        self._stage_ptrs = [None, None]
        self._recv_ptrs = [None, None]
        # flag words: [0:8] ready, [8:16] done (gathering), [16:24] arrival counters, [24:32] done (reducing)
        self._flags = symm_mem.empty(64, dtype=torch.int32, device=device)
        self._flags.zero_()
        self._flag_ptrs = list(symm_mem.rendezvous(self._flags, group).buffer_ptrs)
        self._local = torch.zeros(272, dtype=torch.int32, device=device)   # flags, counters, per-group arrival flags
        self._reduce_state = torch.zeros(4, dtype=torch.int32, device=device)   # [calls completed, arrivals expected]
        # SM budget of the fused kernels: "off" (default) gives every call the whole device. Moving remote data takes
        # SMs as well as link time (about 9 GB/s per pulling or pushing SM), so a transfer-bound call finishes soonest
        # with all of them: on eight ranks, budgets sized by tensor work alone stretched the output projection's
        # GEMM -> reduce-scatter to 1355 us where NCCL's reduce-scatter plus the GEMM take 1000. "auto" (opt-in) gives
        # a call the SMs its products or its transfer need, whichever is more, and leaves the rest to kernels on other
        # streams (weight gradients, a second micro-batch); `sm_cap` bounds it (two fused kernels of two micro-batch
        # streams must fit side by side).
        mode = os.environ.get("AJB_FUSED_SM_BUDGET", "off")
        self.sm_budget_mode = mode if mode in ("auto", "off") else int(mode)
        self.sm_cap: int | None = None
        self._sms = int(native.lib().ajb_sm_count())
        torch.cuda.synchronize(device)
        dist.barrier(group)
        fn = native.lib().ajb_comm_gemm
        fn.argtypes = [ctypes.POINTER(_CommArgs), ctypes.c_void_p]
        fn.restype = ctypes.c_int
        self._fn = fn

    # ------------------------------------------------------------------ symmetric buffers (grown on demand)
    def _ensure(self, which: str, nbytes: int):
        """Both parities of a buffer kind grow together (a collective: every rank reaches the same sizes in the same
        call because the shapes are the same on every rank)."""
        buffers = getattr(self, f"_{which}")
        if buffers[0] is not None and buffers[0].numel() - self.GUARD_BYTES >= nbytes:
            return
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"the symmetric {which} buffer would have to grow to {nbytes} bytes during a graph capture; "
                               "run the step once outside the capture first")
        # Outgrown buffers stay allocated: a CUDA graph captured earlier carries their (and the peers') addresses in its
        # kernel arguments, and every rank replays the same graphs, so such a graph keeps exchanging through the old set
        self._retired.extend(b for b in buffers if b is not None)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        size = max(nbytes, 1 << 20)
        pointers = getattr(self, f"_{which}_ptrs")
        for parity in (0, 1):
            # a guard page behind the payload: peers write into this buffer with raw pointers, and a pattern that
            # survives (`guards_intact`) shows that none of them ran past the end
            buf = self._symm.empty(size + self.GUARD_BYTES, dtype=torch.uint8, device=self.device)
            buf[size:].fill_(self.GUARD_PATTERN)
            pointers[parity] = list(self._symm.rendezvous(buf, self.group).buffer_ptrs)
            buffers[parity] = buf
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def guards_intact(self) -> bool:
        """True when the guard bytes behind every symmetric buffer still hold their pattern."""
        for buf in (*self._stage, *self._recv):
            if buf is not None and not bool((buf[-self.GUARD_BYTES:] == self.GUARD_PATTERN).all()):
                return False
        return True

    def supports(self, rows_total: int) -> bool:
        return rows_total % self.size == 0 and (rows_total // self.size) % self.BLOCK_M == 0

    def _launch(self, mode: int, m: int, n: int, k: int, b: torch.Tensor, b_mn: bool, out: torch.Tensor,
                a: torch.Tensor | None = None, gathered: torch.Tensor | None = None, a_rows: int = 0,
                shard_elems: int = 0, b_offset_elems: int = 0, swiglu: int = 0, aux: torch.Tensor | None = None) -> None:
        gathers = mode in (MODE_ALL_GATHER, MODE_GATHER_WEIGHT)
        parity = self.gather_calls & 1          # gathering: _next_stage() advanced the count and filled this parity
        args = _CommArgs()
        args.mode, args.m, args.n, args.k = mode, m, n, k
        args.tp, args.rank, args.b_mn_major = self.size, self.rank, int(b_mn)
        args.copy_ctas = self.copy_ctas_link_bound if (gathers and self._link_bound(mode, m, n, k)) else self.copy_ctas
        args.ldb, args.ldc = (b.stride(0) if b.dim() == 2 else k), out.stride(0)
        args.shard_elems, args.b_offset_elems = shard_elems, b_offset_elems
        args.a = a.data_ptr() if a is not None else None
        args.b, args.out = b.data_ptr(), out.data_ptr()
        args.gathered = gathered.data_ptr() if gathered is not None else None
        args.a_rows = a_rows
        args.swiglu = swiglu
        args.aux = aux.data_ptr() if aux is not None else None
        args.ld_aux = aux.stride(0) if aux is not None else 0
        for r in range(self.size):
            args.stage_ptrs[r] = self._stage_ptrs[parity][r] if (gathers and self._stage_ptrs[parity]) else None
            args.recv_ptrs[r] = self._recv_ptrs[1][r] if self._recv_ptrs[1] else None
            args.recv_ptrs_even[r] = self._recv_ptrs[0][r] if self._recv_ptrs[0] else None
            args.ready_ptrs[r] = self._flag_ptrs[r]
            args.done_ptrs[r] = self._flag_ptrs[r] + (8 if gathers else 24) * 4
            args.counter_ptrs[r] = self._flag_ptrs[r] + 16 * 4
        args.shard_flags = self._local.data_ptr()
        args.reduce_state = self._reduce_state.data_ptr()
        args.epoch = self.gather_calls & 0xFFFFFFFF
        native.launch_count += 1
        with nvtx_range(("ag_gemm", "gemm_rs", "gemm_ar", "gw_gemm")[mode]), native.sm_budget(self._budget(mode, m, n, k)):
            status = self._fn(ctypes.byref(args), native.stream_ptr())
        if status != 0:
            raise RuntimeError(f"ajb_comm_gemm failed: {native.lib().ajb_last_error().decode()}")

    # measured on this kind of box: peer copies reach about 770 GB/s per direction, cuBLAS-class bf16 GEMMs about
    # 1.39 PFLOP/s sustained
    LINK_BYTES_PER_S, TENSOR_FLOPS = 750e9, 1.3e15

    def _times(self, mode: int, m: int, n: int, k: int) -> tuple[float, float]:
        """(seconds on the link, seconds on the tensor cores) of one fused call at the measured rates."""
        moved = (self.size - 1) / self.size * m * (n if mode == MODE_REDUCE_SCATTER else k) * 2
        if mode == MODE_GATHER_WEIGHT:
            moved = (self.size - 1) / self.size * n * k * 2
        return moved / self.LINK_BYTES_PER_S, 2.0 * m * n * k / self.TENSOR_FLOPS

    def _link_bound(self, mode: int, m: int, n: int, k: int) -> bool:
        link_s, tensor_s = self._times(mode, m, n, k)
        return link_s > tensor_s

    def _budget(self, mode: int, m: int, n: int, k: int) -> int | None:
        """SMs for one fused call (None: the whole device)."""
        if self.sm_budget_mode == "off" or mode == MODE_ALL_REDUCE:
            return self.sm_cap
        if self.sm_budget_mode != "auto":
            want = int(self.sm_budget_mode)
        else:
            link_s, tensor_s = self._times(mode, m, n, k)
            share = min(1.0, 1.3 * tensor_s / max(link_s, 1e-9))      # 30 % headroom over the break-even share
            # the link needs SMs too: one SM pulls or pushes about 9 GB/s of remote data
            floor = (self.copy_ctas_link_bound + 32) if mode != MODE_REDUCE_SCATTER else 96
            want = max(floor, int(self._sms * share) // 2 * 2)
        if self.sm_cap is not None:
            want = min(want, self.sm_cap)
        return None if want >= self._sms - 8 else want

    def _next_stage(self, nbytes: int) -> torch.Tensor:
        """Opens the next gathering call: the staging buffer of its parity, free to overwrite because the previous call
        did not return before every peer had finished reading it (two calls ago)."""
        self._ensure("stage", nbytes)
        self.gather_calls += 1
        return self._stage[self.gather_calls & 1][:nbytes]

    # ------------------------------------------------------------------ raw fused ops
    def all_gather_gemm(self, x_local: torch.Tensor, weight: torch.Tensor, b_mn: bool, n: int, k: int,
                        swiglu: int = 0, aux: torch.Tensor | None = None):
        """Returns ``(gathered [M, k], out [M, n])`` with ``out = gathered @ op(weight)``.

        ``swiglu = 1``: ``out`` holds (gate, up) pairs and the epilogue also writes ``aux [M, n / 2] = silu(gate) * up``.
        ``swiglu = 2``: the product is ``d_act``, ``aux`` is the saved ``gate_up [M, 2 n]`` and ``out [M, 2 n]`` is the
        gradient of the pairs; ``d_act`` is never stored."""
        m_local = x_local.shape[0]
        m = m_local * self.size
        stage = self._next_stage(m_local * k * 2).view(torch.bfloat16).view(m_local, k)
        stage.copy_(x_local)
        gathered = torch.empty(m, k, dtype=torch.bfloat16, device=self.device)
        gathered[self.rank * m_local:(self.rank + 1) * m_local].copy_(x_local)   # the kernel moves only remote shards
        out = torch.empty(m, 2 * n if swiglu == 2 else n, dtype=torch.bfloat16, device=self.device)
        self._launch(MODE_ALL_GATHER, m, n, k, weight, b_mn, out, gathered=gathered, swiglu=swiglu, aux=aux)
        return gathered, out

    def gemm_reduce_scatter(self, x: torch.Tensor, weight: torch.Tensor, b_mn: bool, n: int, k: int) -> torch.Tensor:
        """``reduce_scatter_rows(x @ op(weight))`` -> ``[M / tp, n]``."""
        m = x.shape[0]
        m_local = m // self.size
        self._ensure("recv", self.size * m_local * n * 2)
        out = torch.empty(m_local, n, dtype=torch.bfloat16, device=self.device)
        self._launch(MODE_REDUCE_SCATTER, m, n, k, weight, b_mn, out, a=x)
        return out

    def gemm_all_reduce(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``sum over ranks of x @ weight^T`` -> ``[rows, n]`` on every rank (inference; no autograd).

        Meant for decoding, where ``rows`` is small: every rank's partial tiles are stored into every
        peer's receive buffer by the GEMM epilogue and summed at the end of the same kernel."""
        rows, k = x.shape
        n = weight.shape[0]
        m = -(-rows // self.BLOCK_M) * self.BLOCK_M
        self._ensure("recv", self.size * m * n * 2)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=self.device)
        self._launch(MODE_ALL_REDUCE, m, n, k, weight, False, out, a=x.contiguous(), a_rows=rows)
        return out[:rows]

    def gather_weight_gemm(self, x: torch.Tensor, shard: torch.Tensor, n: int, k: int, offset_elems: int = 0,
                           out_flat: torch.Tensor | None = None):
        """``x @ W^T`` where ``W [n, k]`` starts at element ``offset_elems`` of the flat parameter buffer that is
        the concatenation of every rank's ``shard`` (fully sharded weights; inference or the forward of a unit).

        Returns ``(flat, out)``: the gathered flat buffer (all parameters of the unit, usable by the GEMMs
        that follow; ``out_flat`` when given) and ``out [rows, n]``. The peers' slices travel while the first
        tiles are computed."""
        rows = x.shape[0]
        if rows % self.BLOCK_M != 0 or x.dtype != torch.bfloat16 or shard.dtype != torch.bfloat16:
            raise ValueError("gather_weight_gemm needs bf16 operands and a multiple of 128 rows")
        shard_elems = shard.numel()
        self._next_stage(shard_elems * 2).view(torch.bfloat16).copy_(shard.reshape(-1))
        flat = out_flat if out_flat is not None else torch.empty(self.size * shard_elems, dtype=torch.bfloat16, device=self.device)
        if flat.numel() != self.size * shard_elems or flat.dtype != torch.bfloat16 or not flat.is_contiguous():
            raise ValueError("out_flat must be a contiguous bf16 buffer of world * shard elements")
        flat[self.rank * shard_elems:(self.rank + 1) * shard_elems].copy_(shard.reshape(-1))   # the kernel moves remote slices
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=self.device)
        self._launch(MODE_GATHER_WEIGHT, rows, n, k, flat, False, out, a=x.contiguous(), gathered=flat,
                     shard_elems=shard_elems, b_offset_elems=offset_elems)
        return flat, out

    # ------------------------------------------------------------------ differentiable entry points
    def gather_linear(self, x_local: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        if x_local.dtype != torch.bfloat16 or not self.supports(x_local.shape[0] * self.size):
            from ajllm_b200 import ops
            from ajllm_b200.parallel.tensor_parallel import _GatherRows
            return ops.linear(_GatherRows.apply(x_local, self.group), weight)
        return _GatherLinearFn.apply(x_local, weight, self)

    def linear_scatter(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        if x.dtype != torch.bfloat16 or not self.supports(x.shape[0]):
            from ajllm_b200 import ops
            from ajllm_b200.parallel.tensor_parallel import _ScatterRows
            return _ScatterRows.apply(ops.linear(x, weight), self.group)
        return _LinearScatterFn.apply(x, weight, self)


    def swiglu_ffn(self, x_local: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
        """Sequence-parallel SwiGLU block: all-gather -> W13 GEMM with the activation in its epilogue, then W2 GEMM ->
        reduce-scatter; the backward pass computes the activation gradient in the epilogue of the gathered
        ``d_out @ W2``. ``w13 [2 F_local, D]`` interleaved, ``w2 [D, F_local]``."""
        from ajllm_b200.ops import functional

        f = w13.shape[0] // 2
        if (not functional.FUSED_SWIGLU or x_local.dtype != torch.bfloat16 or f % 32 != 0
                or not self.supports(x_local.shape[0] * self.size)):
            from ajllm_b200 import ops
            return self.linear_scatter(ops.swiglu_interleaved(self.gather_linear(x_local, w13)), w2)
        return _SwigluFfnFn.apply(x_local, w13, w2, self)


def _wgrad(grad_out: torch.Tensor, activations: torch.Tensor, weight: torch.Tensor):
    """``dW[n, k] = grad_out[M, n]^T @ activations[M, k]`` into ``weight.main_grad`` or a new tensor."""
    n, k = weight.shape
    main = getattr(weight, "main_grad", None)
    if main is not None:
        wgrad_accumulate(grad_out, activations, main, n, k, grad_out.shape[0])
        weight.main_grad_written = True
        return None
    out = torch.empty(n, k, dtype=torch.bfloat16, device=grad_out.device)
    gemm(grad_out, activations, out, n, k, grad_out.shape[0], a_mn_major=True, b_mn_major=True)
    return out


class _GatherLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight, fused: FusedTensorParallel):
        n, k = weight.shape
        gathered, out = fused.all_gather_gemm(x_local.contiguous(), weight, False, n, k)
        ctx.save_for_backward(gathered, weight)
        ctx.fused = fused
        return out

    @staticmethod
    def backward(ctx, grad_out):
        gathered, weight = ctx.saved_tensors
        n, k = weight.shape
        grad_out = grad_out.contiguous()
        # dX[M, k] = dY[M, n] @ W[n, k], reduce-scattered to this rank's tokens
        grad_x = ctx.fused.gemm_reduce_scatter(grad_out, weight, True, k, n)
        grad_w = _wgrad(grad_out, gathered, weight) if ctx.needs_input_grad[1] else None
        return grad_x, grad_w, None


class _SwigluFfnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, w13, w2, fused: FusedTensorParallel):
        f2, k = w13.shape
        d_out = w2.shape[0]
        m = x_local.shape[0] * fused.size
        act = torch.empty(m, f2 // 2, dtype=torch.bfloat16, device=x_local.device)
        gathered, gate_up = fused.all_gather_gemm(x_local.contiguous(), w13, False, f2, k, swiglu=1, aux=act)
        out = fused.gemm_reduce_scatter(act, w2, False, d_out, f2 // 2)
        ctx.save_for_backward(gathered, w13, w2, gate_up, act)
        ctx.fused = fused
        return out

    @staticmethod
    def backward(ctx, grad_local):
        gathered, w13, w2, gate_up, act = ctx.saved_tensors
        f2, k = w13.shape
        d_out = w2.shape[0]
        # d_out is gathered over ranks while d_act = d_out @ W2 runs; its epilogue turns d_act into d_gate_up
        grad_full, d_gate_up = ctx.fused.all_gather_gemm(grad_local.contiguous(), w2, True, f2 // 2, d_out, swiglu=2, aux=gate_up)
        grad_w2 = _wgrad(grad_full, act, w2) if ctx.needs_input_grad[2] else None
        grad_x = ctx.fused.gemm_reduce_scatter(d_gate_up, w13, True, k, f2)
        grad_w13 = _wgrad(d_gate_up, gathered, w13) if ctx.needs_input_grad[1] else None
        return grad_x, grad_w13, grad_w2, None


class _LinearScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, fused: FusedTensorParallel):
        n, k = weight.shape
        x = x.contiguous()
        out = fused.gemm_reduce_scatter(x, weight, False, n, k)
        ctx.save_for_backward(x, weight)
        ctx.fused = fused
        return out

    @staticmethod
    def backward(ctx, grad_local):
        x, weight = ctx.saved_tensors
        n, k = weight.shape
        # dY is gathered over ranks while dX[M, k] = dY[M, n] @ W[n, k] runs on the shards already present
        grad_full, grad_x = ctx.fused.all_gather_gemm(grad_local.contiguous(), weight, True, k, n)
        grad_w = _wgrad(grad_full, x, weight) if ctx.needs_input_grad[1] else None
        return grad_x, grad_w, None
