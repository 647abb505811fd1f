"""Graph-captured decode plans.

The reference found real decode to be dispatch-bound, not bandwidth-bound
(jang_tools/dsv41/DECODE_DSPARK_METHODS.md:90-93) and fused its dispatches by
hand.  On CUDA the same effect comes from capturing the launches of a decode
step once and replaying them: `GemvPlan` captures the mat-vecs of its linears on
a private stream into a CUDA graph; `run()` replays it, `run_host()` adds the
host->device copy of the step's activations and the device->host copy of the
last output.  Linears named in one inner list of `groups` read the same
activations (q/k/v, or gate/up, of a decoder layer) and go out through
jq_qgemv_batched_ex, which makes one launch of every run that shares K, the
bit width and the group size.

`persistent=True` goes one step further (the reference's hand-fused dispatches,
dsv41/metal_decode.py:464-497): every run of consecutive groups the streamed
program takes (one activation row, 2-/4-/6-/8-bit codes) becomes ONE cooperative
launch, jq_qgemv_stream_run, whose op boundaries are grid barriers inside the
kernel; groups it does not take (other widths) keep their own launch.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import _lib
from .linear import JANGLinear


class GemvPlan:
    """A fixed sequence of quantized mat-vecs (one per linear), batch `m` rows.

    Every linear has its own input row buffer `x[i]` ([m, in_features]) and
    output buffer `y[i]`; the caller (or `run_host`) fills the inputs.
    """

    def __init__(self, linears: Sequence[JANGLinear], m: int = 1, dtype: torch.dtype = torch.bfloat16,
                 device=None, share_inputs: bool = True, static_weights: bool = True,
                 groups: Sequence[Sequence[int]] | None = None, persistent: bool = False):
        if m < 1 or m > _lib.QGEMV_MAX_M:
            raise _lib.JangqError(_lib.JQ_EINVAL, f"GemvPlan takes 1..{_lib.QGEMV_MAX_M} rows")
        self.linears = list(linears)
        self.m, self.dtype = m, dtype
        # the plan's weights are fixed once it exists, so launches may overlap their predecessors
        self.static_weights = static_weights
        self.device = torch.device(device if device is not None else self.linears[0].weight.device)
        # one input buffer per distinct in_features when sharing (a real decoder reuses the hidden state)
        self._xbuf = {}
        self.x, self.y = [], []
        for lin in self.linears:
            key = lin.in_features if share_inputs else len(self.x)
            if key not in self._xbuf:
                self._xbuf[key] = torch.zeros((m, lin.in_features), dtype=dtype, device=self.device)
            self.x.append(self._xbuf[key])
            self.y.append(torch.empty((m, lin.out_features), dtype=dtype, device=self.device))
        self.algorithmic_bytes = sum(self.bytes_of(lin, m) for lin in self.linears)
        # groups: lists of indices into `linears` whose members share an input; default: every linear alone
        self.groups = [list(g) for g in groups] if groups is not None else [[i] for i in range(len(self.linears))]
        if sorted(i for g in self.groups for i in g) != list(range(len(self.linears))):
            raise _lib.JangqError(_lib.JQ_EINVAL, "groups must name every linear exactly once")
        for g in self.groups:
            if any(self.x[i] is not self.x[g[0]] for i in g):
                raise _lib.JangqError(_lib.JQ_EINVAL, "the linears of a group must read the same input buffer")
        self.launches_per_run = sum(self._launches_of(g) for g in self.groups) * ((m + 7) // 8)
        # persistent: segments = ("program", StreamProgram) or ("groups", [group, ...]) in execution order
        self.persistent = bool(persistent) and m == 1
        self._segments = None
        if self.persistent:
            self._segments, launches, run = [], 0, []
            for g in self.groups + [None]:
                if g is not None and self._streamable(g):
                    run.append(g)
                    continue
                if run:
                    self._segments.append(("program", StreamProgram(
                        [(self.x[r[0]], [self.linears[i] for i in r], [self.y[i] for i in r]) for r in run], dtype)))
                    launches += 1
                    run = []
                if g is not None:
                    self._segments.append(("groups", [g]))
                    launches += self._launches_of(g)
            self.launches_per_run = launches
        self._graph = None
        self._host_in = {k: torch.zeros(v.shape, dtype=dtype).pin_memory() for k, v in self._xbuf.items()}
        self._host_out = torch.zeros(self.y[-1].shape, dtype=dtype).pin_memory()

    @staticmethod
    def bytes_of(lin: JANGLinear, m: int) -> int:
        """Algorithmic bytes of one mat-vec: codes + sidecars + activations in + out."""
        n, k = lin.out_features, lin.in_features
        e = lin.scales.element_size()
        return n * k * lin.bits // 8 + n * (k // lin.group_size) * 2 * e + m * k * 2 + m * n * 2

    def _launches_of(self, group) -> int:
        """Kernel launches of one group: runs of up to 4 consecutive members with equal (K, bits, group size)."""
        n, run, prev = 0, 0, None
        for i in group:
            lin = self.linears[i]
            key = (lin.in_features, lin.bits, lin.group_size)
            if key != prev or run == 4:
                n, run, prev = n + 1, 0, key
            run += 1
        return n

    def _streamable(self, group) -> bool:
        lins = [self.linears[i] for i in group]
        l0 = lins[0]
        return (len(lins) <= 4 and l0.bits in (2, 4, 6, 8) and l0.group_size in (64, 128) and
                l0.in_features % (4 * l0.group_size) == 0 and
                all(l.bits == l0.bits and l.group_size == l0.group_size and l.in_features == l0.in_features and
                    l.scales.dtype == self.dtype and l.bias is None for l in lins))

    def _enqueue(self):
        from .ops import qgemv_fused
        flags = _lib.JQ_GEMV_STATIC_WEIGHTS if self.static_weights else 0
        if self._segments is not None:
            for kind, what in self._segments:
                if kind == "program":
                    what.run()
                else:
                    for g in what:
                        qgemv_fused(self.x[g[0]], [self.linears[i] for i in g], [self.y[i] for i in g], flags)
            return
        for g in self.groups:
            qgemv_fused(self.x[g[0]], [self.linears[i] for i in g], [self.y[i] for i in g], flags)

    def capture(self):
        """Record the launches into a CUDA graph (call once, before run())."""
        with torch.cuda.device(self.device):
            s = torch.cuda.Stream(self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                self._enqueue()            # warm-up outside capture (sets function attributes)
            torch.cuda.current_stream(self.device).wait_stream(s)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue()
            self._graph = g
        return self

    def run(self):
        """Replay on the current stream (falls back to direct launches before capture())."""
        if self._graph is None:
            self._enqueue()
        else:
            self._graph.replay()
        return self.y

    def check_status(self):
        """Raise JangqError(JQ_ETIMEOUT) if a bounded device-side wait of a launch ran out since the last check (the
        outputs of that run are undefined).  Reads the device status word, which synchronises the device: call it at
        step boundaries of a serving loop, not between launches."""
        _lib.check(_lib.load().jq_device_status())

    def run_host(self, host_inputs: dict | None = None) -> torch.Tensor:
        """One step from host memory: pinned inputs -> device, replay, last output -> pinned host."""
        src = host_inputs if host_inputs is not None else self._host_in
        for k, buf in self._xbuf.items():
            buf.copy_(src[k], non_blocking=True)
        self.run()
        self._host_out.copy_(self.y[-1], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self._host_out

    @property
    def h2d_bytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self._xbuf.values())

    @property
    def d2h_bytes(self) -> int:
        return self._host_out.numel() * self._host_out.element_size()


class StreamProgram:
    """A prepared program of dependent one-row mat-vecs for jq_qgemv_stream_run: `ops` is a list of
    (x [1, K] or [K], [linear, ...], [y, ...]) in execution order; the linears of an op share x, K, the bit
    width (2, 4, 6 or 8) and the group size.  An op with more rows than one op of a program may have is cut
    into row ranges (consecutive ops over slices of the same tensors).  The program keeps references to the
    tensors it names; run() enqueues the one launch on the current stream."""

    MAX_TILES_PER_CTA = 14          # row tiles per SM an op may have (the kernel's limit of 16 minus both ends)

    def __init__(self, ops, dtype: torch.dtype = torch.bfloat16):
        import ctypes as C
        lib = _lib.load()
        self._keep = ops
        first = ops[0][0]
        self.device = first.device
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        flat = []
        for x, lins, ys in ops:
            l0 = lins[0]
            tiles = sum((l.out_features + 15) // 16 for l in lins)
            parts = max(1, -(-tiles // (self.MAX_TILES_PER_CTA * sms)))
            if parts == 1:
                flat.append((x, [(l.weight, l.scales, l.biases, y.reshape(-1)) for l, y in zip(lins, ys)], l0))
                continue
            for l, y in zip(lins, ys):          # too many rows: every matrix on its own, in row chunks
                n = l.out_features
                chunk = -(-n // (parts * 16)) * 16
                for r0 in range(0, n, chunk):
                    r1 = min(n, r0 + chunk)
                    flat.append((x, [(l.weight[r0:r1], l.scales[r0:r1], l.biases[r0:r1], y.reshape(-1)[r0:r1])], l0))
        self.n_ops = len(flat)
        arr = (_lib.JqStreamOp * self.n_ops)()
        for d, (x, mats, l0) in zip(arr, flat):
            d.x = x.data_ptr()
            d.K, d.bits, d.group_size, d.count = l0.in_features, l0.bits, l0.group_size, len(mats)
            for i, (w, s, b, y) in enumerate(mats):
                d.codes[i], d.scales[i], d.biases[i], d.y[i], d.N[i] = (w.data_ptr(), s.data_ptr(), b.data_ptr(),
                                                                          y.data_ptr(), w.shape[0])
        nbytes = int(lib.jq_qgemv_stream_workspace_bytes(arr, self.n_ops))
        self.workspace = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=self.device)
        self.program = _lib.JqStreamProgram()
        with torch.cuda.device(self.device):
            _lib.check(lib.jq_qgemv_stream_prepare(arr, self.n_ops, _lib.dtype_id(dtype), self.workspace.data_ptr(),
                                                   self.workspace.numel(), C.byref(self.program),
                                                   _lib.stream_ptr(self.device)))

    def run(self):
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().jq_qgemv_stream_run(self.program, _lib.stream_ptr(self.device)))
