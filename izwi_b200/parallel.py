"""Sharding of the hot path over the GPUs of one box: tensor-parallel projections with one
all-reduce per block, expert-parallel MoE with an all-to-all each way, batch-parallel encoders.

The partition arithmetic is plain Python / NumPy so it can be tested on CPU ranks; the data path
uses the C ABI (izb_comm_*, izb_tp_allreduce, izb_ep_alltoall) and the CUDA kernels.  The
reference is single-device, so none of this mirrors reference code.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

# ----------------------------------------------------------------------------------------------
# partition arithmetic (no torch, no GPU)
# ----------------------------------------------------------------------------------------------


def split_range(n: int, parts: int, index: int) -> tuple[int, int]:
    """Contiguous block `index` of `n` items cut into `parts` near-equal blocks (first blocks larger)."""
    if parts <= 0 or not 0 <= index < parts:
        raise ValueError("bad partition index")
    base, rem = divmod(n, parts)
    lo = index * base + min(index, rem)
    return lo, lo + base + (1 if index < rem else 0)


def tp_qkv_rows(q_heads: int, kv_heads: int, head_dim: int, tp: int, rank: int) -> np.ndarray:
    """Rows of the fused [q; k; v] weight that rank `rank` owns: its query heads and the kv heads
    they attend with (kv heads are replicated when tp exceeds their number)."""
    if q_heads % tp != 0:
        raise ValueError(f"{q_heads} query heads do not split {tp} ways")
    qh = q_heads // tp
    q_rows = np.arange(rank * qh * head_dim, (rank + 1) * qh * head_dim)
    if kv_heads % tp == 0:
        kh = kv_heads // tp
        kv = np.arange(rank * kh * head_dim, (rank + 1) * kh * head_dim)
    elif tp % kv_heads == 0:
        head = rank // (tp // kv_heads)
        kv = np.arange(head * head_dim, (head + 1) * head_dim)
    else:
        raise ValueError(f"{kv_heads} kv heads do not split or replicate {tp} ways")
    q_total, kv_total = q_heads * head_dim, kv_heads * head_dim
    return np.concatenate([q_rows, q_total + kv, q_total + kv_total + kv])


def tp_gate_up_rows(intermediate: int, tp: int, rank: int) -> np.ndarray:
    """Rows of the fused [gate; up] weight for a rank: gate_i and up_i of the same columns stay together."""
    lo, hi = split_range(intermediate, tp, rank)
    return np.concatenate([np.arange(lo, hi), intermediate + np.arange(lo, hi)])


def tp_row_split_cols(k: int, tp: int, rank: int) -> tuple[int, int]:
    """Input columns of a row-split (O / down) projection owned by a rank."""
    return split_range(k, tp, rank)


def ep_expert_range(n_experts: int, ep: int, rank: int) -> tuple[int, int]:
    """Experts [lo, hi) living on a rank: contiguous blocks."""
    if n_experts % ep != 0:
        raise ValueError(f"{n_experts} experts do not split {ep} ways")
    per = n_experts // ep
    return rank * per, (rank + 1) * per


def ep_send_rows(offsets: np.ndarray, ep: int) -> np.ndarray:
    """Rows this rank sends to each rank, from its permuted-row offsets [E+1] (rows are ordered by
    expert, so the rows of one destination are contiguous)."""
    e = len(offsets) - 1
    per = e // ep
    return np.array([int(offsets[(r + 1) * per] - offsets[r * per]) for r in range(ep)], dtype=np.int64)


def ep_recv_plan(all_offsets: np.ndarray, ep: int, rank: int) -> tuple[np.ndarray, np.ndarray]:
    """From every rank's offsets [ep, E+1]: rows received from each rank, and the local expert id
    of every received row in arrival order (source-major, expert-minor)."""
    e = all_offsets.shape[1] - 1
    lo, hi = ep_expert_range(e, ep, rank)
    counts = np.diff(all_offsets, axis=1)[:, lo:hi]              # [src, local expert]
    recv_rows = counts.sum(axis=1).astype(np.int64)
    local_ids = np.concatenate([np.repeat(np.arange(hi - lo), counts[s]) for s in range(ep)]) if counts.sum() else \
        np.zeros(0, np.int64)
    return recv_rows, local_ids.astype(np.int32)


def ep_peer_tables(counts: np.ndarray, rank: int) -> dict:
    """The placement tables of the peer-memory dispatch (izb_ep_dispatch derives the same on the
    device from the exchanged counts).  counts [world, E]: rows rank s holds for expert e.
      dst_row[e]       first row, in the owner's receive buffer, of this rank's rows for expert e
      recv_start[l, s] first received row of (local expert l, source s); rows are grouped by local
                       expert, then source rank, then source order
      seg[l]           grouped-GEMM offsets over the local experts (seg[-1] = rows received)
      ret_start[s, l]  row, in source s's own expert-major order, where its rows of local expert l begin
    """
    world, e = counts.shape
    per = e // world
    dst_row = np.zeros(e, dtype=np.int64)
    for ex in range(e):
        first = ex // per * per
        dst_row[ex] = counts[:, first:ex].sum() + counts[:rank, ex].sum()
    mine = counts[:, rank * per:(rank + 1) * per]                  # [source, local expert]
    flat = mine.T.reshape(-1)                                      # local expert major, source minor
    starts = np.concatenate([[0], np.cumsum(flat)])
    recv_start = starts[:-1].reshape(per, world)
    seg = np.concatenate([recv_start[:, 0], [starts[-1]]])
    src_offsets = np.concatenate([np.zeros((world, 1), dtype=np.int64), np.cumsum(counts, axis=1)], axis=1)
    ret_start = src_offsets[:, rank * per:(rank + 1) * per]
    return {"dst_row": dst_row, "recv_start": recv_start, "seg": seg, "ret_start": ret_start, "total": int(starts[-1])}


def batch_split(batch: int, world: int, rank: int) -> tuple[int, int]:
    """Utterances [lo, hi) a rank encodes (weights replicated, no collective)."""
    return split_range(batch, world, rank)


# ----------------------------------------------------------------------------------------------
# NCCL communicator over the C ABI
# ----------------------------------------------------------------------------------------------


class Comm:
    """izb_comm built from an initialised torch.distributed group (used only to pass the id)."""

    def __init__(self, device_index: int):
        import torch
        import torch.distributed as dist

        from . import _lib as L
        from .ops import Context
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.ctx = Context.get(device_index)
        ident = torch.zeros(128, dtype=torch.uint8)
        if self.rank == 0:
            buf = (C.c_ubyte * 128)()
            L.check(L.lib().izb_comm_unique_id(buf), "izb_comm_unique_id")
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        ident = ident.to(torch.device("cuda", device_index))
        dist.broadcast(ident, src=0)
        raw = bytes(ident.cpu().tolist())
        handle = C.c_void_p()
        L.check(L.lib().izb_comm_init(self.ctx.handle, self.world, self.rank, raw, C.byref(handle)), "izb_comm_init")
        self.handle = handle

    def allreduce_(self, t):
        import torch

        from . import _lib as L
        from .ops import _ptr, _stream
        assert t.is_contiguous()
        code = L.IZB_F32 if t.dtype == torch.float32 else L.IZB_BF16
        nbytes = t.numel() * t.element_size()
        big = nbytes > (1 << 20)          # two-shot path: 16-byte aligned operand (a ragged end takes the one-shot kernel)
        if getattr(self, "ar", None) and nbytes <= self.ar_max and nbytes % 4 == 0 \
                and t.data_ptr() % (16 if big else 4) == 0:
            L.check(L.lib().izb_ar_allreduce(self.ar, _stream(), _ptr(t), t.numel(), code), "izb_ar_allreduce")
        else:
            L.check(L.lib().izb_tp_allreduce(self.handle, _stream(), _ptr(t), t.numel(), code), "izb_tp_allreduce")
        return t

    def allgather_bytes(self, send, recv):
        from . import _lib as L
        from .ops import _ptr, _stream
        L.check(L.lib().izb_comm_allgather(self.handle, _stream(), _ptr(send), _ptr(recv),
                                           send.numel() * send.element_size()), "izb_comm_allgather")

    def alltoall_rows(self, send, send_rows, recv, recv_rows, row_bytes: int):
        from . import _lib as L
        from .ops import _ptr, _stream
        s = (C.c_int64 * self.world)(*[int(v) for v in send_rows])
        r = (C.c_int64 * self.world)(*[int(v) for v in recv_rows])
        L.check(L.lib().izb_ep_alltoall(self.handle, _stream(), _ptr(send), s, _ptr(recv), r, row_bytes),
                "izb_ep_alltoall")

    def enable_peer_allreduce(self, max_bytes: int = 1 << 20):
        """Sets up the all-reduce over NVLink peer memory for messages up to max_bytes (one-shot up to
        1 MB, two-shot above); larger ones keep going through NCCL.  Also creates the second stream on
        which `allreduce_async_` / `reduce_region_async` run the sums.  Collective: every rank must call it."""
        import torch
        import torch.distributed as dist

        from . import _lib as L
        ar = C.c_void_p()
        L.check(L.lib().izb_ar_create(self.ctx.handle, self.world, self.rank, max_bytes, C.byref(ar)), "izb_ar_create")
        mine = (C.c_ubyte * 64)()
        L.check(L.lib().izb_ar_local_handle(ar, mine), "izb_ar_local_handle")
        every = [None] * self.world
        dist.all_gather_object(every, bytes(mine))
        L.check(L.lib().izb_ar_connect(ar, b"".join(every)), "izb_ar_connect")
        dist.barrier()
        self.ar, self.ar_max = ar, max_bytes
        self.side = torch.cuda.Stream(device=self.ctx.device)
        self._pending = []            # events of sums still running on the side stream
        self._region_done = [None, None]

    # -- sums that overlap the next projection: issued on the side stream, joined by the caller --
    # Events are kept with a note of whether they were recorded while the stream was being captured into
    # a CUDA graph.  A capture may only wait on events of the same capture (torch synchronises the device
    # before capturing, so earlier work is complete anyway), and eager code must not wait on events that
    # exist only inside a graph (replays are ordered on their stream as a whole).
    @staticmethod
    def _record(stream):
        import torch
        ev = torch.cuda.Event()
        ev.record(stream)
        return (ev, torch.cuda.is_current_stream_capturing())

    @staticmethod
    def wait_for(marked):
        """The current stream waits for an event returned by allreduce_async_ / kept by this class."""
        import torch
        ev, captured = marked
        if captured == torch.cuda.is_current_stream_capturing():
            torch.cuda.current_stream().wait_event(ev)

    def _fork(self):
        import torch
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.side.wait_event(ev)

    def allreduce_async_(self, t):
        """allreduce_(t) on the side stream, after everything issued so far on the current stream.
        The current stream sees the sum after `join()`, or after waiting for the returned event."""
        import torch
        self._fork()
        with torch.cuda.stream(self.side):
            self.allreduce_(t)
            ev = self._record(self.side)
        self._pending.append(ev)
        return ev

    def region_ok(self, n_elems: int, elem_size: int = 2) -> bool:
        """Whether a sum of this size can take the copy-free two-shot path through the region."""
        nbytes = n_elems * elem_size
        return bool(getattr(self, "ar", None)) and (1 << 20) < nbytes <= self.ar_max and nbytes % 16 == 0

    def region_views(self, which: int, rows: int, cols: int):
        """(operand, result) bf16 [rows, cols] views of two-shot buffer `which` inside this rank's region."""
        import torch

        from . import _lib as L

        class _Raw:
            def __init__(self, ptr, n):
                self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<u2", "data": (ptr, False), "version": 2}
        n = rows * cols
        dev = torch.device("cuda", self.ctx.device)
        op = torch.as_tensor(_Raw(L.lib().izb_ar_operand(self.ar, which), n), device=dev).view(torch.bfloat16).view(rows, cols)
        res = torch.as_tensor(_Raw(L.lib().izb_ar_result(self.ar, which), n), device=dev).view(torch.bfloat16).view(rows, cols)
        return op, res

    def wait_region_free(self, which: int):
        """The current stream waits until the previous sum on buffer `which` has completed (its operand
        may then be rewritten)."""
        ev = self._region_done[which]
        if ev is not None:
            self.wait_for(ev)

    def reduce_region_async(self, which: int, n_elems: int):
        """Sums buffer `which` over the ranks on the side stream, after everything issued so far on the
        current stream (the projection that wrote the operand)."""
        import torch

        from . import _lib as L
        self._fork()
        with torch.cuda.stream(self.side):
            L.check(L.lib().izb_ar_allreduce_region(self.ar, C.c_void_p(self.side.cuda_stream), which, n_elems, L.IZB_BF16),
                    "izb_ar_allreduce_region")
            ev = self._record(self.side)
        self._region_done[which] = ev
        self._pending.append(ev)

    def reset_events(self):
        """Forgets the recorded events after a device-wide synchronise (call between a run that was
        captured into a CUDA graph and the next capture: events of an ended capture cannot be waited on)."""
        import torch
        torch.cuda.synchronize()
        self._pending = []
        self._region_done = [None, None]

    def join(self):
        """The current stream waits for every sum issued on the side stream so far."""
        for ev in self._pending:
            self.wait_for(ev)
        self._pending = []

    def enable_peer_ep(self, n_experts: int, hidden: int, max_tokens_local: int, top_k: int):
        """Sets up expert-parallel dispatch / return over NVLink peer memory (izb_ep_*) for layers of
        this shape and at most max_tokens_local tokens per rank and step.  Collective."""
        import torch.distributed as dist

        from . import _lib as L
        ep = C.c_void_p()
        L.check(L.lib().izb_ep_create(self.ctx.handle, self.world, self.rank, n_experts, hidden, max_tokens_local, top_k,
                                      C.byref(ep)), "izb_ep_create")
        mine = (C.c_ubyte * 64)()
        L.check(L.lib().izb_ep_local_handle(ep, mine), "izb_ep_local_handle")
        every = [None] * self.world
        dist.all_gather_object(every, bytes(mine))
        L.check(L.lib().izb_ep_connect(ep, b"".join(every)), "izb_ep_connect")
        dist.barrier()
        self.ep = ep
        self.ep_shape = (n_experts, hidden, max_tokens_local, top_k)

    def close(self):
        from . import _lib as L
        if getattr(self, "ep", None):
            L.lib().izb_ep_destroy(self.ep)
            self.ep = None
        if getattr(self, "ar", None):
            L.lib().izb_ar_destroy(self.ar)
            self.ar = None
        if self.handle:
            L.lib().izb_comm_destroy(self.handle)
            self.handle = None


# ----------------------------------------------------------------------------------------------
# sharded layers (GPU)
# ----------------------------------------------------------------------------------------------


class TpDecoderLayer:
    """Linear stack of one decoder layer under tensor parallelism: column-split QKV, row-split O with
    an all-reduce, column-split gate/up (pairs kept together) with SwiGLU, row-split down with an
    all-reduce.  Attention itself is outside this path: O takes the rank's slice of its input."""

    def __init__(self, comm: Comm | None, w_qkv, w_o, w_gate_up, w_down, overlap: bool = True):
        self.comm = comm
        # overlap: run the sums on the communicator's side stream, concurrently with the projections that
        # follow them.  In this linear-stack workload nothing inside a step consumes a sum (attention
        # and norms are outside it), so the caller joins at the end of the step (comm.join()); a full
        # decoder layer would consume the O sum before gate/up and must join there instead.
        self.overlap = overlap
        self.w_qkv, self.w_o, self.w_gate_up, self.w_down = w_qkv, w_o, w_gate_up, w_down
        self.inter_local = w_gate_up.shape[0] // 2

    @classmethod
    def from_full(cls, comm, shape, w_qkv, w_o, w_gate_up, w_down, tp: int, rank: int, overlap: bool = True):
        import torch
        dev = w_qkv.device
        rows = torch.from_numpy(tp_qkv_rows(shape.q_heads, shape.kv_heads, shape.head_dim, tp, rank)).to(dev)
        gu = torch.from_numpy(tp_gate_up_rows(shape.intermediate, tp, rank)).to(dev)
        olo, ohi = tp_row_split_cols(w_o.shape[1], tp, rank)
        dlo, dhi = tp_row_split_cols(w_down.shape[1], tp, rank)
        return cls(comm, w_qkv[rows].contiguous(), w_o[:, olo:ohi].contiguous(), w_gate_up[gu].contiguous(),
                   w_down[:, dlo:dhi].contiguous(), overlap=overlap)

    def collective_name(self, m: int) -> str:
        """Which sum the O and down outputs of `m` token rows go through."""
        comm = self.comm
        if comm is None:
            return "none"
        nbytes = m * self.w_o.shape[0] * 2
        if getattr(comm, "ar", None) and nbytes <= comm.ar_max:
            return ("izb_ar_allreduce over NVLink peer memory, "
                    + ("one-shot (8-byte {payload, sequence} stores)" if nbytes <= (1 << 20) else "two-shot (reduce-scatter + all-gather)"))
        return "izb_tp_allreduce (NCCL)"

    def forward(self, x_attn_in, x_o_in, x_mlp_in):
        """x_attn_in [M, H] -> qkv_local; x_o_in [M, K_o/tp] -> attention block output (reduced);
        x_mlp_in [M, H] -> MLP block output (reduced)."""
        from . import ops
        m = x_mlp_in.shape[0]
        if m <= 32:
            return self._forward_decode(x_attn_in, x_o_in, x_mlp_in)
        comm = self.comm
        h = self.w_o.shape[0]
        if comm is not None and self.overlap and comm.region_ok(m * h):
            # The row-split projections write their partial sums straight into this rank's peer-mapped
            # region and the sums run on the side stream (one kernel each, two buffers), so the sum of O
            # overlaps the gate/up projection and the sum of down overlaps the next layer's QKV and O.
            # The returned o / down are views of the region, valid after comm.join().
            op0, res0 = comm.region_views(0, m, h)
            op1, res1 = comm.region_views(1, m, h)
            qkv = ops.linear(x_attn_in, self.w_qkv)
            comm.wait_region_free(0)
            ops.linear(x_o_in, self.w_o, out=op0)
            comm.reduce_region_async(0, m * h)
            hidden = ops.linear(x_mlp_in, self.w_gate_up, epilogue="swiglu")
            comm.wait_region_free(1)
            ops.linear(hidden, self.w_down, out=op1)
            comm.reduce_region_async(1, m * h)
            return qkv, res0, res1
        qkv = ops.linear(x_attn_in, self.w_qkv)
        o = ops.linear(x_o_in, self.w_o)
        if comm is not None:
            comm.allreduce_(o)
        hidden = ops.linear(x_mlp_in, self.w_gate_up, epilogue="swiglu")
        down = ops.linear(hidden, self.w_down)
        if comm is not None:
            comm.allreduce_(down)
        return qkv, o, down

    def _forward_decode(self, x_attn_in, x_o_in, x_mlp_in):
        """Decode sizes: the three projections that do not depend on one another go out as one grouped
        persistent launch, then SiLU-multiply, then the down projection; plans and output buffers are
        built once per set of input buffers and reused every step."""
        import torch

        from . import ops
        key = (x_attn_in.data_ptr(), x_o_in.data_ptr(), x_mlp_in.data_ptr(), x_mlp_in.shape[0])
        st = getattr(self, "_decode_state", None)
        if st is None or st["key"] != key:
            dev, m = x_mlp_in.device, x_mlp_in.shape[0]
            mk = lambda n: torch.empty(m, n, device=dev, dtype=torch.bfloat16)  # noqa: E731
            qkv, o, gu = mk(self.w_qkv.shape[0]), mk(self.w_o.shape[0]), mk(self.w_gate_up.shape[0])
            hidden, down = mk(self.inter_local), mk(self.w_down.shape[0])
            first = ops.LinearGroup([
                ops.linear_args(x_attn_in, self.w_qkv, "bf16", *self.w_qkv.shape, qkv),
                ops.linear_args(x_o_in, self.w_o, "bf16", *self.w_o.shape, o),
                ops.linear_args(x_mlp_in, self.w_gate_up, "bf16", *self.w_gate_up.shape, gu)], dev)
            second = ops.LinearGroup([ops.linear_args(hidden, self.w_down, "bf16", *self.w_down.shape, down)], dev)
            st = self._decode_state = dict(key=key, qkv=qkv, o=o, gu=gu, hidden=hidden, down=down, first=first,
                                           second=second, keep=(x_attn_in, x_o_in, x_mlp_in))
        comm = self.comm
        overlap = comm is not None and self.overlap and getattr(comm, "side", None) is not None
        if overlap:
            # this layer's previous sums (the step before) still own the buffers this step rewrites
            for ev in st.get("events", ()):
                comm.wait_for(ev)
            st["events"] = []
        st["first"].launch()
        if comm is not None:
            if overlap:
                st["events"].append(comm.allreduce_async_(st["o"]))
            else:
                comm.allreduce_(st["o"])
        ops.silu_mul(st["gu"][:, : self.inter_local], st["gu"][:, self.inter_local:], out=st["hidden"])
        st["second"].launch()
        if comm is not None:
            if overlap:
                st["events"].append(comm.allreduce_async_(st["down"]))
            else:
                comm.allreduce_(st["down"])
        return st["qkv"], st["o"], st["down"]


class EpMoeLayer:
    """MoE feed-forward layer with the experts spread over ranks in contiguous blocks; tokens are
    data-parallel, the router is replicated.  Rows travel to the rank that owns their expert,
    are regrouped by local expert there, and travel back for the weighted combine."""

    def __init__(self, comm: Comm, w_router, router_bias, w_gate_up_local, w_down_local, n_experts: int, top_k: int):
        self.comm = comm
        self.w_router, self.router_bias = w_router, router_bias
        self.w_gate_up, self.w_down = w_gate_up_local.contiguous(), w_down_local.contiguous()
        self.E, self.k = n_experts, top_k
        self.H = w_router.shape[1]
        self.E_local = self.w_gate_up.shape[0]

    def forward(self, x):
        import torch

        from . import moe, ops
        dev, ep, rank = x.device, self.comm.world, self.comm.rank
        t = x.shape[0]
        self.logits, idx, wts = moe.route(x, self.w_router, self.router_bias, self.k)   # logits kept for checks
        offsets, perm, inv = moe.permute(idx, self.E)
        if getattr(self.comm, "ep", None) is not None and self.comm.ep_shape[:2] == (self.E, self.H) \
                and self.comm.ep_shape[3] == self.k and t <= self.comm.ep_shape[2] and x.stride(1) == 1:
            return self._forward_peer(x, perm, offsets, inv, wts, idx, t)
        x_perm = moe.gather(x, perm, self.k)
        # routing counts of every rank (the row counts of the exchange must be known on the host)
        all_off = torch.empty(ep, self.E + 1, device=dev, dtype=torch.int32)
        self.comm.allgather_bytes(offsets, all_off)
        all_off_h = all_off.cpu().numpy()
        send_rows = ep_send_rows(all_off_h[rank], ep)
        recv_rows, local_ids = ep_recv_plan(all_off_h, ep, rank)
        r_total = int(recv_rows.sum())
        recv = torch.empty(max(r_total, 1), self.H, device=dev, dtype=torch.bfloat16)
        self.comm.alltoall_rows(x_perm, send_rows, recv, recv_rows, self.H * 2)
        if r_total > 0:
            ids = torch.from_numpy(local_ids).to(dev)
            l_off, l_perm, l_inv = moe.permute(ids, self.E_local)
            xs = moe.gather(recv, l_perm, 1)
            hid = moe.grouped_gemm(xs, self.w_gate_up, l_off, "swiglu")
            ys = moe.grouped_gemm(hid, self.w_down, l_off)
            back = moe.gather(ys, l_inv, 1)            # arrival order again
        else:
            back = recv
        y_perm = torch.empty(max(t * self.k, 1), self.H, device=dev, dtype=torch.bfloat16)
        self.comm.alltoall_rows(back, recv_rows, y_perm, send_rows, self.H * 2)
        return moe.combine(y_perm[: t * self.k], inv, wts), idx, wts

    def _forward_peer(self, x, perm, offsets, inv, wts, idx, t):
        """Dispatch (with the gather fused in) and return through peer memory: no host read."""
        import torch

        from . import _lib as L
        from . import moe
        from .ops import Context, _ptr, _stream
        lib, ep, dev = L.lib(), self.comm.ep, x.device
        ctx = Context.get(dev.index)
        cap = lib.izb_ep_recv_capacity_rows(ep)
        inter = self.w_down.shape[2]
        if getattr(self, "_peer_bufs", None) is None or self._peer_bufs[0].shape[0] != cap:
            self._peer_bufs = (torch.empty(cap, inter, device=dev, dtype=torch.bfloat16),
                               torch.empty(cap, self.H, device=dev, dtype=torch.bfloat16))
        hid, ys = self._peer_bufs
        L.check(lib.izb_ep_dispatch(ep, _stream(), _ptr(x), x.stride(0), _ptr(perm), _ptr(offsets), t * self.k),
                "izb_ep_dispatch")
        recv, seg = C.c_void_p(lib.izb_ep_recv_rows(ep)), C.c_void_p(lib.izb_ep_recv_offsets(ep))
        L.check(lib.izb_moe_grouped_gemm(ctx.handle, _stream(), recv, _ptr(self.w_gate_up), seg, _ptr(hid), L.IZB_BF16, cap,
                                         2 * inter, self.H, self.E_local, moe.EPILOGUE["swiglu"]), "izb_moe_grouped_gemm")
        L.check(lib.izb_moe_grouped_gemm(ctx.handle, _stream(), _ptr(hid), _ptr(self.w_down), seg, _ptr(ys), L.IZB_BF16, cap,
                                         self.H, inter, self.E_local, moe.EPILOGUE[None]), "izb_moe_grouped_gemm")
        L.check(lib.izb_ep_return(ep, _stream(), _ptr(ys)), "izb_ep_return")
        y = torch.empty(t, self.H, device=dev, dtype=torch.bfloat16)
        L.check(lib.izb_moe_combine(ctx.handle, _stream(), C.c_void_p(lib.izb_ep_returned_rows(ep)), _ptr(inv), _ptr(wts), t,
                                    self.k, self.H, _ptr(y)), "izb_moe_combine")
        return y, idx, wts
