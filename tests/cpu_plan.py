"""Test infrastructure: executes a ``Plan`` on the CPU with the oracle's arithmetic.

It exists to check HOST logic without a GPU — that the recogniser, the fusion passes and the
tensor-parallel decoder plans describe the right computation — by running the plan's operator
list against numpy buffers. It is never imported by the package; the product path always goes
through the native library.
"""

from __future__ import annotations

import math

import numpy as np

from oracle import reference_ops as R

_ITEMSIZE = {"f32": 4, "bf16": 2, "f16": 2, "i32": 4, "i64": 8}


class CpuPlanRunner:
    """Buffers are flat float64/int arrays (one per slot) holding values already rounded to
    the slot's dtype; views are gathered / scattered with explicit strides."""

    def __init__(self, plan, allreduce=None, rank=0, world=1):
        self.plan = plan
        self.allreduce = allreduce  # callable(np.ndarray) -> np.ndarray (sum over ranks), for TP tests
        self.rank, self.world = rank, world
        self.bufs: list[np.ndarray] = []

    # -- views -------------------------------------------------------------------------------
    @staticmethod
    def _index(view) -> np.ndarray:
        idx = np.full(view.shape, view.offset, dtype=np.int64)
        for d, (n, s) in enumerate(zip(view.shape, view.strides)):
            shp = [1] * len(view.shape)
            shp[d] = n
            idx = idx + (np.arange(n, dtype=np.int64) * s).reshape(shp)
        return idx

    def read(self, view) -> np.ndarray:
        return self.bufs[view.slot][self._index(view)]

    def write(self, view, values) -> None:
        values = np.asarray(values)
        if view.dtype in ("i32", "i64"):
            out = values.astype(np.int64)
        else:
            out = R.round_to(values.astype(np.float32), view.dtype).astype(np.float64)
        self.bufs[view.slot][self._index(view)] = out.reshape(view.shape)

    # -- execution ------------------------------------------------------------------------------
    def run(self, args: list[np.ndarray]) -> list[np.ndarray]:
        plan = self.plan
        assert len(args) == len(plan.args)
        self.bufs = []
        for a, spec in zip(args, plan.args):
            assert tuple(a.shape) == tuple(spec.shape), (a.shape, spec.shape, spec.name)
            flat = np.asarray(a).reshape(-1)
            self.bufs.append(flat.astype(np.int64) if spec.dtype in ("i32", "i64") else flat.astype(np.float64))
        for nbytes in plan.temp_bytes:
            self.bufs.append(np.full(nbytes // 2 + 8, np.nan))  # poison: reads of unwritten temporaries show up
        self._reset_clocks()
        for op in plan.ops:
            self._check_ordering(op)
            getattr(self, "_" + op.kind)(op)
        return [self.bufs[i].reshape(spec.shape) for i, spec in enumerate(plan.args)]

    def _gemm(self, op):
        d, a, b, c, bias, res = op.operands[:6]
        flags = op.attrs.get("flags", 0)
        A, B = self.read(a).astype(np.float32), self.read(b).astype(np.float32)
        acc = A @ B
        if flags & 4:  # SwiGLU: column blocks [gate 128 | up 128]
            n = acc.shape[-1]
            blocks = acc.reshape(acc.shape[0], n // 256, 2, 128)
            acc = (R.silu(blocks[:, :, 0, :]) * blocks[:, :, 1, :]).reshape(acc.shape[0], n // 2)
        if c is not None:
            acc = acc + self.read(c).astype(np.float32)
        if bias is not None:
            acc = acc + self.read(bias).astype(np.float32)
        acc = R.ACTIVATIONS[op.attrs.get("act", "none")](acc)
        if res is not None:
            acc = acc + self.read(res).astype(np.float32)
        self.write(d, acc)

    def _gemm_rope(self, op):
        d, a, b = op.operands[:3]
        at = op.attrs
        acc = R.round_to(self.read(a).astype(np.float32) @ self.read(b).astype(np.float32), d.dtype)
        cols, hd, seq = at["rope_cols"], at["head_dim"], at["seq"]
        if cols:
            x = acc[:, :cols].reshape(acc.shape[0] // seq, seq, cols // hd, hd)
            acc[:, :cols] = R.rope(x, at["theta"], at["pos0"], d.dtype).reshape(acc.shape[0], cols)
        self.write(d, acc)

    def _attention(self, op):
        o, q, k, v = op.operands[:4]
        Q, K, V = self.read(q), self.read(k), self.read(v)
        if Q.ndim == 3:
            Q, K, V = Q[:, None], K[:, None], V[:, None]
        out = R.attention(Q, K, V, scale=op.attrs["scale"], causal=op.attrs.get("causal", False), io_dtype=q.dtype)
        self.write(o, out.reshape(o.shape))

    def _layernorm(self, op):
        out, x, g, b = op.operands[:4]
        self.write(out, R.layernorm(self.read(x), None if g is None else self.read(g), None if b is None else self.read(b), op.attrs["eps"]))

    def _rmsnorm(self, op):
        out, x, w = op.operands[:3]
        self.write(out, R.rmsnorm(self.read(x), None if w is None else self.read(w), op.attrs["eps"], out.dtype))

    def _softmax(self, op):
        self.write(op.operands[0], R.softmax(self.read(op.operands[1])))

    def _rope(self, op):
        x = op.operands[0]
        self.write(x, R.rope(self.read(x), op.attrs["theta"], op.attrs["pos0"], x.dtype))

    def _elementwise(self, op):
        out, a, b = op.operands[:3]
        kind, act, s = op.attrs["ew"], op.attrs.get("act", "none"), op.attrs.get("scalar", 0.0)
        A = None if a is None else np.broadcast_to(self.read(a).astype(np.float32), out.shape)
        B = None if b is None else np.broadcast_to(self.read(b).astype(np.float32), out.shape)
        f = R.ACTIVATIONS[act]
        val = {
            "copy": lambda: A, "add": lambda: A + B, "mul": lambda: A * B, "sub": lambda: A - B, "max": lambda: np.maximum(A, B),
            "act": lambda: f(A), "add_act": lambda: f(A + B), "silu_mul": lambda: R.silu(A) * B,
            "scale": lambda: A * np.float32(s), "fill": lambda: np.full(out.shape, s, np.float32),
        }[kind]()
        self.write(out, val)

    def _embedding(self, op):
        out, ids, wte, wpe = op.operands[:4]
        idv = self.read(ids).reshape(-1)
        val = self.read(wte)[idv]
        if wpe is not None:
            val = val + self.read(wpe)[np.arange(idv.size) % op.attrs["period"]]
        self.write(out, val.reshape(out.shape))

    def _allreduce(self, op):
        v = op.operands[0]
        if self.allreduce is not None:
            self.write(v, self.allreduce(self.read(v)))

    def _reducescatter(self, op):
        out, inp = op.operands[:2]
        total = self.read(inp) if self.allreduce is None else self.allreduce(self.read(inp))
        flat = np.asarray(total).reshape(self.world, -1)
        self.write(out, flat[self.rank].reshape(out.shape))

    def _allgather(self, op):
        out, inp = op.operands[:2]
        mine = self.read(inp)
        if self.world == 1:
            self.write(out, mine.reshape(out.shape))
            return
        full = np.zeros((self.world,) + mine.shape)
        full[self.rank] = mine
        self.write(out, self.allreduce(full).reshape(out.shape))  # a gather as a sum of disjoint blocks

    def _reduce_norm_gather(self, op):
        xn, part, h, w = op.operands[:4]
        rows = h.shape[0]
        mine = slice(self.rank * rows, (self.rank + 1) * rows)
        hv = self.read(h)
        if part is not None:
            parts = R.round_to(self.read(part).astype(np.float32), "bf16").astype(np.float64)
            total = parts if self.allreduce is None else self.allreduce(parts)
            total = R.round_to(np.asarray(total, dtype=np.float32), "bf16")  # the switch returns the activation type
            hv = hv.astype(np.float32) + total[mine]
            self.write(h, hv)
            hv = self.read(h)
        normed = R.round_to(R.rmsnorm(hv, self.read(w), op.attrs["eps"], xn.dtype).astype(np.float32), xn.dtype)
        full = np.zeros(xn.shape)
        full[mine] = normed
        self.write(xn, full if self.world == 1 else self.allreduce(full))

    # -- two streams -------------------------------------------------------------------------
    # The interpreter runs both streams in program order, which every correctly synchronised
    # plan allows, and checks the synchronisation itself with vector clocks: two accesses to
    # one slot from different streams, at least one of them a write, must be ordered by events.
    _WRITES = {"gemm": 1, "gemm_rope": 1, "attention": 1, "layernorm": 1, "rmsnorm": 1, "softmax": 1, "rope": 1, "elementwise": 1,
               "embedding": 1, "allreduce": 1, "allgather": 1, "reducescatter": 1, "reduce_norm_gather": 1}

    def _reset_clocks(self):
        self.cur = 0
        self.clock = [[0, 0], [0, 0]]  # clock[s][t]: how many operators of stream t stream s has seen
        self.event_clock: dict[int, list[int]] = {}
        self.last_write: dict[int, tuple[int, int, str]] = {}
        self.reads: dict[int, list[tuple[int, int, str]]] = {}

    def _ordered(self, access) -> bool:
        stream, count, _ = access
        return self.clock[self.cur][stream] >= count

    def _check_ordering(self, op):
        if op.kind not in self._WRITES:
            return
        self.clock[self.cur][self.cur] += 1
        me = (self.cur, self.clock[self.cur][self.cur], op.kind)
        views = [v for v in op.operands if v is not None]
        out_slot = views[0].slot
        for v in views[1:] + ([views[0]] if op.kind in ("rope", "allreduce") else []):
            w = self.last_write.get(v.slot)
            assert w is None or self._ordered(w), f"{op.kind} on stream {self.cur} reads slot {v.slot} without waiting for {w[2]} on stream {w[0]}"
        w = self.last_write.get(out_slot)
        assert w is None or self._ordered(w), f"{op.kind} on stream {self.cur} overwrites slot {out_slot} without waiting for {w[2]} on stream {w[0]}"
        for r in self.reads.get(out_slot, []):
            assert self._ordered(r), f"{op.kind} on stream {self.cur} overwrites slot {out_slot} still read by {r[2]} on stream {r[0]}"
        for v in views[1:]:
            if v.slot != out_slot:
                self.reads.setdefault(v.slot, []).append(me)
        self.last_write[out_slot] = me
        self.reads[out_slot] = []
        if op.kind == "reduce_norm_gather":  # also updates the residual rows (operand 2)
            self.last_write[op.operands[2].slot] = me
            self.reads[op.operands[2].slot] = []

    def _stream(self, op):
        self.cur = op.attrs["index"]

    def _event_record(self, op):
        self.event_clock[op.attrs["index"]] = list(self.clock[self.cur])

    def _event_wait(self, op):
        assert op.attrs["index"] in self.event_clock, f"event {op.attrs['index']} waited for before its record"
        seen = self.event_clock[op.attrs["index"]]
        self.clock[self.cur] = [max(a, b) for a, b in zip(self.clock[self.cur], seen)]

    def _reserve_sms(self, op):
        pass
