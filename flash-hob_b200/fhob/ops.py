"""Host side of the B200 double-backward flash attention operator.

Mirrors the reference entry point
``flash_bwdbwd(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale) -> (dQ2, dK2, dV2, ddO)``
(fhog/triton_bwdbwd.py:557-648) on top of the C ABI of libfhob.so.  torch is
used for device memory and streams only; all arithmetic runs in the library's
CUDA kernels, and a missing library is an error rather than a fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib

_workspaces: dict = {}


def _workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    if torch.cuda.is_current_stream_capturing():
        # memory allocated while a CUDA graph is captured belongs to the graph's pool: the graph
        # keeps it alive for its replays, a cache that outlives the graph must not
        return torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _fold(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dim() == 4:
        t = t.reshape(t.shape[0] * t.shape[1], t.shape[2], t.shape[3])
    if t.dim() != 3:
        raise ValueError(f"{name}: expected (BH, N, D) or (B, H, N, D), got {tuple(t.shape)}")
    return t.contiguous()


def _tc_capable(dtype: torch.dtype, d: int, d_v: int) -> bool:
    """Shapes the tensor-core kernels take (they are the ones that read views through tensor maps)."""
    if dtype == torch.float32:
        return d <= 64 and d_v <= 64 and d % 4 == 0 and d_v % 4 == 0
    return d <= 128 and d_v <= 128 and d % 8 == 0 and d_v % 8 == 0


def _strides_of(t: torch.Tensor, batches: int, heads: int):
    """(row, head, batch) element strides of a (BH, N, D) or (B, H, N, D) tensor over the common
    (batches, heads) split of the folded axis, or None when the tensor cannot be read in place:
    last dim not contiguous, a stride or the base address off the 16-byte grid, heads of the folded
    axis not equally spaced."""
    align = 16 // t.element_size()
    if t.data_ptr() % 16 or (t.shape[-1] > 1 and t.stride(-1) != 1):
        return None
    if t.dim() == 4:
        if tuple(t.shape[:2]) != (batches, heads):
            return None
        batch, head, row = t.stride(0), t.stride(1), t.stride(2)
    else:
        if t.shape[0] != batches * heads:
            return None
        head, row = t.stride(0), t.stride(1)
        batch = head * heads
    if t.shape[-2] == 1:
        row = t.shape[-1]          # a single row: any positive stride describes it
    if row <= 0 or head < 0 or batch < 0 or row % align or head % align or batch % align:
        return None
    return row, head, batch


def _window(is_causal, sliding_window) -> int:
    """0 for no window, else the validated sliding_window_length."""
    if sliding_window is None or sliding_window == float("inf"):
        return 0
    w = int(sliding_window)
    if w != sliding_window or w < 1 or w > 2 ** 31 - 1:
        raise ValueError(f"sliding_window must be a positive integer, got {sliding_window!r}")
    if not is_causal:
        raise ValueError("sliding_window needs is_causal=True (the window trails the causal diagonal)")
    return w


class _Problem:
    """Validated tensors + the FhobProblem struct that points at them."""

    def __init__(self, Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, is_causal, impl, need_outputs=True,
                 window=None, out=None, workspace=None, allow_views=True):
        names = ("Q", "K", "V", "O", "dO", "ddQ", "ddK", "ddV")
        no_o = O is None
        if no_o:
            O = dO   # stands in for the shape checks; the library gets a NULL pointer
        tensors = [Q, K, V, O, dO, ddQ, ddK, ddV]
        if impl not in _lib.IMPL:
            raise ValueError(f"impl must be one of {sorted(_lib.IMPL)}, got {impl!r}")
        for n, t in zip(names, tensors):
            if not isinstance(t, torch.Tensor):
                raise TypeError(f"{n} must be a torch.Tensor")
        dev, dt = Q.device, Q.dtype
        if dev.type != "cuda":
            raise ValueError("device tensors expected (use flash_bwdbwd, which stages host tensors)")
        if str(dt) not in _lib.DTYPES:
            raise TypeError(f"dtype {dt} not supported: bfloat16, float16 or float32")
        for n, t in zip(names, tensors):
            if t.device != dev:
                raise ValueError(f"{n} is on {t.device}, Q is on {dev}")
            if t.dtype != dt:
                raise TypeError(f"{n} has dtype {t.dtype}, Q has {dt}")
        self.out_shapes = (Q.shape, K.shape, V.shape, dO.shape)   # dQ2, dK2, dV2, ddO
        for n, t in zip(names, tensors):
            if t.dim() not in (3, 4):
                raise ValueError(f"{n}: expected (BH, N, D) or (B, H, N, D), got {tuple(t.shape)}")
        # Views (a (B, N, H, D) projection seen as (B, H, N, D), a slice of a fused QKV tensor, ...)
        # are read in place through tensor maps when the tensor-core kernels run and every stride
        # stays on the 16-byte grid; anything else is made contiguous first (a copy).
        batches, heads = (Q.shape[0], Q.shape[1]) if Q.dim() == 4 else (1, Q.shape[0])
        strides = None
        if (allow_views and impl != "simt" and _tc_capable(dt, Q.shape[-1], V.shape[-1])
                and not all(t.is_contiguous() for t in tensors)):
            strides = [_strides_of(t, batches, heads) for t in tensors]
            if any(st is None for st in strides):
                strides = None
        if strides is None:
            t3 = [_fold(t, n) for n, t in zip(names, tensors)]
        else:
            # shape-only stand-ins (folded) for the checks below; the kernels read `tensors` in place
            t3 = [torch.empty((t.shape[0] if t.dim() == 3 else t.shape[0] * t.shape[1], t.shape[-2], t.shape[-1]),
                              dtype=dt, device="meta") for t in tensors]
        q, k, v, o, do, ddq, ddk, ddv = t3
        bh, n_q, d = q.shape
        n_k, d_v = k.shape[1], v.shape[2]
        # two head dims (jax_refs/flash_impl.py:381-389): Q, K and their cotangents share one, V, O, dO, ddV the other
        want_shapes = dict(Q=(bh, n_q, d), ddQ=(bh, n_q, d), K=(bh, n_k, d), ddK=(bh, n_k, d),
                           V=(bh, n_k, d_v), ddV=(bh, n_k, d_v), O=(bh, n_q, d_v), dO=(bh, n_q, d_v))
        for n, t in zip(names, t3):
            if tuple(t.shape) != want_shapes[n]:
                raise ValueError(f"{n}: shape {tuple(t.shape)} does not match {want_shapes[n]}")
        lse = L.reshape(-1, L.shape[-1]) if L.dim() >= 2 else L.reshape(1, -1)
        if tuple(lse.shape) != (bh, n_q) or L.device != dev:
            raise ValueError(f"L: expected {(bh, n_q)} on {dev}, got {tuple(L.shape)} on {L.device}")
        lse = lse.to(torch.float32).contiguous()
        self.keep = (t3 if strides is None else tensors) + [lse]
        self.device = dev
        self.stream = torch.cuda.current_stream(dev).cuda_stream
        lib = _lib.load()
        p = _lib.FhobProblem()
        p.bh, p.n_q, p.n_k, p.d = bh, n_q, n_k, d
        p.d_v = 0 if d_v == d else d_v
        p.dtype = _lib.DTYPES[str(dt)]
        p.causal = 1 if is_causal else 0
        p.window = _window(is_causal, window)
        p.impl = _lib.IMPL[impl]
        p.scale = float(scale)
        if workspace is None:
            # what lets the library take its fastest path (fp32 with head dim 64: room for the bf16
            # hi/lo copies of the inputs, so that the problem runs on the tensor cores)
            self.ws = _workspace(dev, self.stream, lib.fhob_workspace_bytes_problem(C.byref(p)))
        else:
            nbytes = lib.fhob_workspace_bytes(bh, n_q)
            if (workspace.device != dev or workspace.dtype != torch.uint8 or not workspace.is_contiguous()
                    or workspace.numel() < nbytes or workspace.data_ptr() % 256):
                raise ValueError(f"workspace: need a contiguous uint8 tensor of at least {nbytes} bytes on {dev}, "
                                 "256-byte aligned")
            self.ws = workspace
        src = tensors if strides is not None else t3      # views: the caller's tensors, read in place
        p.q, p.k, p.v, p.o, p.d_o, p.ddq, p.ddk, p.ddv = (t.data_ptr() for t in src)
        if no_o:
            p.o = None
        p.lse = lse.data_ptr()
        self.layout = None
        if strides is not None:
            lay = _lib.FhobLayout()
            lay.heads = heads
            for i, (row, head, batch) in enumerate(strides):
                lay.row[i], lay.head[i], lay.batch[i] = row, head, batch
            lay.lse_head, lay.lse_batch = n_q, heads * n_q
            self.layout = lay                              # kept alive with the problem
            p.layout = C.pointer(lay)
        if need_outputs and out is not None:
            want = (torch.Size((bh, n_q, d)), torch.Size((bh, n_k, d)), torch.Size((bh, n_k, d_v)),
                    torch.Size((bh, n_q, d_v)))
            if len(out) != 4:
                raise ValueError("out: expected (dQ2, dK2, dV2, ddO)")
            folded = []
            for n, t, w_shape in zip(("dQ2", "dK2", "dV2", "ddO"), out, want):
                if t.device != dev or t.dtype != dt or not t.is_contiguous() or t.numel() != w_shape.numel():
                    raise ValueError(f"out {n}: need a contiguous {dt} tensor of {tuple(w_shape)} elements on {dev}")
                folded.append(t.view(w_shape))
            self.dq2, self.dk2, self.dv2, self.ddo = folded
            p.dq2, p.dk2, p.dv2, p.ddo = (t.data_ptr() for t in (self.dq2, self.dk2, self.dv2, self.ddo))
        elif need_outputs:
            new = lambda n, w: torch.empty(bh, n, w, dtype=dt, device=dev)   # results are always contiguous
            self.dq2, self.ddo = new(n_q, d), new(n_q, d_v)
            self.dk2, self.dv2 = new(n_k, d), new(n_k, d_v)
            p.dq2, p.dk2, p.dv2, p.ddo = (t.data_ptr() for t in (self.dq2, self.dk2, self.dv2, self.ddo))
        p.workspace, p.workspace_bytes = self.ws.data_ptr(), self.ws.numel()
        self.p = p
        self.bh, self.n_q = bh, n_q

    def outputs(self):
        return tuple(t.reshape(s) for t, s in zip((self.dq2, self.dk2, self.dv2, self.ddo), self.out_shapes))

    def status(self) -> int:
        """Synchronises the stream and returns the device status word."""
        return _lib.load().fhob_read_status(C.byref(self.p), C.c_void_p(self.stream))


def _run_device(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, is_causal, impl, check, window=None, out=None,
                workspace=None):
    prob = _Problem(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, is_causal, impl, window=window, out=out,
                    workspace=workspace)
    lib = _lib.load()
    with torch.cuda.device(prob.device):
        rc = lib.fhob_bwdbwd(C.byref(prob.p), C.c_void_p(prob.stream))
        if rc != 0 and prob.layout is not None:
            # a view the driver's tensor-map encoder (or the library) does not take: fall back to copies
            prob = _Problem(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, is_causal, impl, window=window, out=out,
                            workspace=workspace, allow_views=False)
            rc = lib.fhob_bwdbwd(C.byref(prob.p), C.c_void_p(prob.stream))
        _lib.check(rc, "fhob_bwdbwd")
        if check:
            _lib.check(prob.status(), "fhob_bwdbwd (device status)")
    return prob.outputs()


def _empty_problem(Q, K, V, dO, out):
    """An empty batch, no queries or no keys: nothing is launched.  Sums over no keys (or no
    queries) are zero, so every result that has any element is zero - the same definition as for
    queries without a visible key under a causal mask.  (The reference cannot launch such a
    problem: its grids would have no blocks.)"""
    if out is not None:
        for t in out:
            t.zero_()
        return tuple(out)
    return tuple(torch.zeros_like(t) for t in (Q, K, V, dO))


def flash_bwdbwd(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, *, is_causal: bool = False,
                 sliding_window: Optional[int] = None, impl: str = "auto", check: Optional[bool] = None,
                 device: Optional[torch.device] = None, out=None, workspace=None) -> Tuple[torch.Tensor, ...]:
    """Double backward of scaled-dot-product attention.

    Same positional signature and return order as the reference
    (fhog/triton_bwdbwd.py:558, :648).  Tensors are ``(BH, N, D)`` like the
    reference or ``(B, H, N, D)``; bfloat16 or float16 (tensor-core kernels,
    fp32 accumulation) or float32 (tensor cores with every operand split into
    a bf16 hi + lo pair when D = 64, CUDA-core kernels otherwise).  ``V``, ``O``, ``dO``
    and ``ddV`` may have a head dim of their own (the reference operator has a
    single D, :577; its maths does not need that, jax_refs/flash_impl.py:381-389):
    ``dV2`` and ``ddO`` then have it too; the tensor-core kernels take head dims
    any head dims up to 128 that are multiples of 8.  ``L`` is the logsumexp of
    the masked scaled scores, any float dtype (used as fp32).  ``O`` may be
    ``None`` for 16-bit inputs on the tensor-core path: ``D = rowsum(dO * O)``
    (reference :580) is then replaced by the mathematically equal
    ``sum_j P_ij dP_ij``, which the row-statistics sweep accumulates anyway.

    Keyword-only additions, all behaviour-preserving by default:
    ``is_causal`` bottom-right aligned causal mask (the reference operator has
    none; its oracle does: jax_refs/flash_impl.py:86-91); ``sliding_window``
    the oracle's ``sliding_window_length`` W (needs ``is_causal``): query i
    then sees only the W keys that end at its causal diagonal; ``impl`` one of
    "auto", "simt", "tcgen05"; ``check`` read the device status word after
    the kernels and raise if a bounded device wait ran out.  Reading it
    synchronises the stream, so the default is ``False`` for device tensors
    (the call stays asynchronous; a wait that ran out - which only a hardware
    or driver fault can cause - would then go unnoticed and leave wrong
    results) and ``True`` for host tensors, where the call synchronises anyway;
    ``out`` a tuple ``(dQ2, dK2, dV2, ddO)`` of preallocated contiguous tensors
    to write into and ``workspace`` a uint8 device tensor of
    ``fhob_workspace_bytes`` bytes (the reference allocates both per call,
    :581-584, :617-618; with them given a device call allocates nothing).

    With ``is_causal`` and N_K < N_Q the first N_Q - N_K queries see no key:
    their dQ2 and ddO rows are zero and their rows of ``O`` and ``L`` are not
    read (the reference leaves this case undefined).

    Host (CPU) tensors are accepted too: they are staged to ``device``
    (default: current CUDA device) in head ranges, preferably from pinned
    memory, and the four results come back as pinned host tensors (or in
    ``out``, four host tensors, preferably pinned) after a stream synchronise.
    """
    if Q.numel() == 0 or K.numel() == 0 or V.numel() == 0:
        return _empty_problem(Q, K, V, dO, out)
    if Q.device.type == "cuda":
        return _run_device(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, is_causal, impl, bool(check), sliding_window,
                           out, workspace)
    if not torch.cuda.is_available():
        raise RuntimeError("flash_bwdbwd needs a CUDA device; there is no CPU implementation")
    if workspace is not None:
        raise ValueError("workspace= is only supported for device tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return _run_host((Q, K, V, O, dO, ddQ, ddK, ddV), L, scale, is_causal, impl, check is None or bool(check), dev,
                     window=sliding_window, out=out)


_copy_streams: dict = {}
_staging: dict = {}     # (device, heads per range, shapes) -> ring of device staging sets of the host-buffer path
HOST_STAGES = 3
HOST_RANGE_BYTES = 192 << 20   # input bytes staged per head range on the host-buffer path (measured best of 48-768 MB)


def _host_ranges(bh: int, head_bytes: int, range_bytes: int):
    """Boundaries of the head ranges of the host-buffer path: ranges of about ``range_bytes`` of
    input, at least four when there are that many heads.  What follows the last upload (its kernels
    and its download) is not overlapped with anything, so the last range is cut into a half and
    two quarters to keep that tail short."""
    per_range = max(1, range_bytes // max(1, head_bytes))
    n_chunks = max(-(-bh // per_range), min(bh, 4))
    bounds = [(bh * i) // n_chunks for i in range(n_chunks + 1)]
    lo_last, hi_last = bounds[-2], bounds[-1]
    if n_chunks >= 4 and hi_last - lo_last >= 4:
        q = (hi_last - lo_last) // 4
        bounds[-1:] = [hi_last - 2 * q, hi_last - q, hi_last]
    return bounds


def _run_host(mats, L, scale, is_causal, impl, check, dev, window=None, out=None, range_bytes=None):
    """Host tensors in, pinned host tensors out.  Heads are independent, so the batch is cut into
    head ranges of about ``HOST_RANGE_BYTES`` of input each (at least four ranges when there are
    that many heads) that flow through three streams: upload of range i+1, the kernels of range i
    and the download of range i-1 overlap.  Device staging memory is a ring of three sets of
    buffers kept per device and shape, so after the first call of a shape nothing is allocated on
    the device; the results' pinned buffers come from torch's caching host allocator (or ``out=``)."""
    names = ("Q", "K", "V", "O", "dO", "ddQ", "ddK", "ddV")
    out_shapes = (mats[0].shape, mats[1].shape, mats[2].shape, mats[4].shape)   # dQ2, dK2, dV2, ddO
    mats3 = [None if t is None else _fold(t, n) for t, n in zip(mats, names)]   # O may be None (not uploaded then)
    bh = mats3[0].shape[0]
    lse = (L.reshape(-1, L.shape[-1]) if L.dim() >= 2 else L.reshape(1, -1)).to(torch.float32)
    if lse.shape[0] != bh:
        raise ValueError(f"L: expected {bh} rows, got {tuple(L.shape)}")
    want = (mats3[0], mats3[1], mats3[2], mats3[4])
    if out is None:
        outs_host = [torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True) for t in want]
    else:
        if len(out) != 4:
            raise ValueError("out: expected (dQ2, dK2, dV2, ddO)")
        outs_host = []
        for n, t, w in zip(("dQ2", "dK2", "dV2", "ddO"), out, want):
            if t.device.type != "cpu" or t.dtype != w.dtype or not t.is_contiguous() or t.numel() != w.numel():
                raise ValueError(f"out {n}: need a contiguous host {w.dtype} tensor of {tuple(w.shape)} elements")
            outs_host.append(t.view(w.shape))
    main = torch.cuda.current_stream(dev)
    up, down = _copy_streams.setdefault(dev.index, (torch.cuda.Stream(dev), torch.cuda.Stream(dev)))
    up.wait_stream(main)
    head_bytes = sum(t[0].numel() * t.element_size() for t in mats3 if t is not None) + lse[0].numel() * 4
    bounds = _host_ranges(bh, head_bytes, int(range_bytes or HOST_RANGE_BYTES))
    n_chunks = len(bounds) - 1
    widest = max(hi - lo for lo, hi in zip(bounds, bounds[1:]))
    sizing = _lib.FhobProblem()       # the widest range decides the workspace (fp32: room for the bf16 copies too)
    sizing.bh, sizing.n_q, sizing.n_k, sizing.d = widest, mats3[0].shape[1], mats3[1].shape[1], mats3[0].shape[2]
    sizing.d_v = 0 if mats3[2].shape[2] == mats3[0].shape[2] else mats3[2].shape[2]
    sizing.dtype, sizing.impl = _lib.DTYPES[str(mats3[0].dtype)], _lib.IMPL[impl]
    ws = _workspace(dev, main.cuda_stream, _lib.load().fhob_workspace_bytes_problem(C.byref(sizing)))
    # Device staging: a ring of HOST_STAGES sets of buffers (nine inputs and four results of the widest
    # range), kept per device and shape, so that a call allocates nothing on the device and the
    # pipeline's timing does not depend on the state of the caching allocator.  Set s is reused by
    # range i + HOST_STAGES once the kernels that read its inputs and the download of its results are done.
    key = (dev.index, widest, tuple(None if t is None else (tuple(t.shape[1:]), t.dtype) for t in mats3))
    ring = _staging.get(key)
    if ring is None:
        if len(_staging) >= 4:
            _staging.clear()
        ring = []
        for _ in range(min(HOST_STAGES, n_chunks)):
            ins = [None if t is None else torch.empty((widest,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
                   for t in mats3]
            ins.append(torch.empty((widest, lse.shape[1]), dtype=torch.float32, device=dev))
            res = [torch.empty((widest,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev) for t in want]
            ring.append(dict(ins=ins, res=res, read=None, drained=None))
        _staging[key] = ring
    for st in ring:
        # a previous call may still be using the set on other streams
        st["read"] = st["drained"] = None
    up.wait_stream(down)
    # the pre-pass of every range clears the status word, so each range's word is kept (on the device:
    # a small device-to-host copy per range would queue behind the downloads on the copy engine)
    status_dev = torch.zeros(n_chunks, dtype=torch.int32, device=dev) if check else None
    for i, (lo, hi) in enumerate(zip(bounds, bounds[1:])):
        st, n = ring[i % len(ring)], hi - lo
        with torch.cuda.stream(up):
            if st["read"] is not None:
                up.wait_event(st["read"])
            for src, dst in zip(mats3 + [lse], st["ins"]):
                if src is not None:
                    dst[:n].copy_(src[lo:hi], non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(up)
        main.wait_event(ready)
        if st["drained"] is not None:
            main.wait_event(st["drained"])
        res = _run_device(*(None if t is None else t[:n] for t in st["ins"]), scale, is_causal, impl, False, window,
                          out=tuple(t[:n] for t in st["res"]), workspace=ws)
        if check:
            status_dev[i:i + 1].copy_(ws[:4].view(torch.int32), non_blocking=True)
        st["read"] = torch.cuda.Event()
        st["read"].record(main)
        down.wait_event(st["read"])
        with torch.cuda.stream(down):
            for h, r in zip(outs_host, res):
                h[lo:hi].copy_(r.reshape(h[lo:hi].shape), non_blocking=True)
            st["drained"] = torch.cuda.Event()
            st["drained"].record(down)
    down.synchronize()
    if check:
        main.synchronize()
        for status in status_dev.tolist():
            _lib.check(status, "fhob_bwdbwd (device status)")
    return tuple(t.reshape(s) for t, s in zip(outs_host, out_shapes))


def release_cached_memory() -> None:
    """Drops the per-stream workspaces and the staging sets of the host-buffer path (device memory
    this module keeps between calls so that repeated calls allocate nothing).  Call it with no
    operator call in flight."""
    torch.cuda.synchronize()
    _workspaces.clear()
    _staging.clear()


def attention_forward(Q, K, V, scale=None, *, is_causal: bool = False, sliding_window: Optional[int] = None,
                      impl: str = "auto", check: bool = False, need_o: bool = True):
    """O(N)-memory producer of the saved forward results: returns ``(O, L)``.

    ``O = softmax(Q K^T scale) V`` in the input dtype and the fp32 logsumexp
    ``L`` — the two tensors ``flash_bwdbwd`` consumes.  Role of the reference's
    forward kernel and ``produce_L`` (fhog/triton_flash.py:12-133, :252-258),
    which is dense, returns L in the input dtype and raises for causal masks.
    16-bit inputs with head dims up to 128, multiples of 8 (V may have its own), and fp32
    inputs with head dim 64 (split into bf16 hi + lo pairs) run on the tensor
    cores (one sweep over the keys with an online softmax), everything else on
    CUDA cores.
    ``need_o=False`` skips the ``P V`` product and returns ``(None, L)``.
    ``check`` synchronises and raises if a bounded device wait ran out.
    Queries that see no key (causal with N_K < N_Q) get ``O = 0``, ``L = -inf``.
    """
    shape_q = Q.shape
    if Q.device.type != "cuda" or str(Q.dtype) not in _lib.DTYPES:
        raise ValueError("attention_forward needs CUDA bfloat16/float16/float32 tensors")
    if impl not in _lib.IMPL:
        raise ValueError(f"impl must be one of {sorted(_lib.IMPL)}, got {impl!r}")
    # views are read in place when the tensor-core kernels run (see _Problem); else folded copies
    strides = None
    if (all(t.dim() in (3, 4) for t in (Q, K, V)) and impl != "simt" and _tc_capable(Q.dtype, Q.shape[-1], V.shape[-1])
            and not all(t.is_contiguous() for t in (Q, K, V))):
        batches, heads = (Q.shape[0], Q.shape[1]) if Q.dim() == 4 else (1, Q.shape[0])
        strides = [_strides_of(t, batches, heads) for t in (Q, K, V)]
        if any(st is None for st in strides):
            strides = None
    if strides is None:
        q, k, v = _fold(Q, "Q"), _fold(K, "K"), _fold(V, "V")
    else:
        q, k, v = (torch.empty((t.shape[0] if t.dim() == 3 else t.shape[0] * t.shape[1], t.shape[-2], t.shape[-1]),
                               dtype=t.dtype, device="meta") for t in (Q, K, V))
    bh, n_q, d = q.shape
    d_v = v.shape[2]
    if k.shape != (bh, k.shape[1], d) or v.shape[:2] != k.shape[:2]:
        raise ValueError(f"K {tuple(k.shape)} / V {tuple(v.shape)} do not match Q {tuple(q.shape)}")
    if scale is None:
        scale = d ** -0.5
    if bh == 0 or n_q == 0 or k.shape[1] == 0 or d == 0 or d_v == 0:
        # nothing to launch; without keys a query has O = 0 and L = -inf, like one the mask leaves without keys
        o = torch.zeros(bh, n_q, d_v, dtype=Q.dtype, device=Q.device) if need_o else None
        lse = torch.full((bh, n_q), float("-inf"), dtype=torch.float32, device=Q.device)
        return (o.reshape(*shape_q[:-1], d_v) if need_o else None), lse.reshape(shape_q[:-1])
    o = torch.empty(bh, n_q, d_v, dtype=Q.dtype, device=Q.device) if need_o else None
    lse = torch.empty(bh, n_q, dtype=torch.float32, device=Q.device)
    p = _lib.FhobProblem()
    p.bh, p.n_q, p.n_k, p.d = bh, n_q, k.shape[1], d
    p.d_v = 0 if d_v == d else d_v
    p.dtype = _lib.DTYPES[str(Q.dtype)]
    p.causal, p.impl, p.scale = (1 if is_causal else 0), _lib.IMPL[impl], float(scale)
    p.window = _window(is_causal, sliding_window)
    src = (Q, K, V) if strides is not None else (q, k, v)
    p.q, p.k, p.v = (t.data_ptr() for t in src)
    lay = None
    if strides is not None:
        lay = _lib.FhobLayout()
        lay.heads = Q.shape[1] if Q.dim() == 4 else bh
        for i, (row, head, batch) in enumerate(strides):
            lay.row[i], lay.head[i], lay.batch[i] = row, head, batch
        p.layout = C.pointer(lay)
    stream = torch.cuda.current_stream(Q.device).cuda_stream
    lib = _lib.load()
    # receives the status word; fp32 with head dim 64: also the bf16 hi/lo copies of the inputs that
    # let the problem run on the tensor cores
    p.n_k = k.shape[1]
    ws = _workspace(Q.device, stream, max(256, lib.fhob_workspace_bytes_problem(C.byref(p))))
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(Q.device):
        call = lambda: lib.fhob_forward(C.byref(p), C.c_void_p(o.data_ptr() if need_o else None),
                                        C.c_void_p(lse.data_ptr()), C.c_void_p(stream))
        rc = call()
        if rc != 0 and lay is not None:
            # a view the tensor-map encoder does not take: read copies instead
            q, k, v = _fold(Q, "Q"), _fold(K, "K"), _fold(V, "V")
            p.q, p.k, p.v, p.layout = q.data_ptr(), k.data_ptr(), v.data_ptr(), None
            rc = call()
        _lib.check(rc, "fhob_forward")
        if check:
            _lib.check(lib.fhob_read_status(C.byref(p), C.c_void_p(stream)), "fhob_forward (device status)")
    return (o.reshape(*shape_q[:-1], d_v) if need_o else None), lse.reshape(shape_q[:-1])


def produce_L(Q, K, is_causal: bool = False, scale=None, sliding_window: Optional[int] = None):
    """fp32 logsumexp of the scaled scores, same name and argument order as the
    reference helper (fhog/triton_flash.py:252-258) but O(N) memory, fp32 and
    causal-capable.  Only the scores are computed (no ``P V`` product)."""
    return attention_forward(Q, K, K, scale, is_causal=is_causal, sliding_window=sliding_window, need_o=False)[1]


def run_passes(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, *, is_causal=False, sliding_window=None, impl="auto",
               upto=4, fused12=False):
    """Runs the pre-pass and passes 1..``upto`` one by one (unit tests, profiling).

    ``fused12`` replaces passes 1 and 2 by the single sweep that ``flash_bwdbwd``
    uses on the tensor-core path (``fhob_pass12``).

    Returns a dict with the row statistics ``d``, ``dd``, ``b`` (fp32, (BH, N_Q));
    entries a pass has not produced yet are garbage), the outputs produced so
    far, and the device ``status`` word.
    """
    prob = _Problem(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, is_causal, impl, window=sliding_window)
    lib = _lib.load()
    s = C.c_void_p(prob.stream)
    with torch.cuda.device(prob.device):
        _lib.check(lib.fhob_prepass(C.byref(prob.p), s), "fhob_prepass")
        stages = [str(i) for i in range(1, upto + 1)]
        if fused12:
            if upto < 2:
                raise ValueError("fused12 needs upto >= 2")
            stages = ["12"] + stages[2:]
        for i in stages:
            _lib.check(getattr(lib, f"fhob_pass{i}")(C.byref(prob.p), s), f"fhob_pass{i}")
        vecs = torch.empty(3, prob.bh, prob.n_q, dtype=torch.float32, device=prob.device)
        _lib.check(lib.fhob_row_stats(C.byref(prob.p), C.c_void_p(vecs[0].data_ptr()),
                                      C.c_void_p(vecs[1].data_ptr()), C.c_void_p(vecs[2].data_ptr()), s),
                   "fhob_row_stats")
        status = prob.status()
    out = dict(d=vecs[0], dd=vecs[1], b=vecs[2], status=status)
    if upto >= 3:
        out["dq2"], out["ddo"] = prob.dq2, prob.ddo
    if upto >= 4:
        out["dk2"], out["dv2"] = prob.dk2, prob.dv2
    return out
