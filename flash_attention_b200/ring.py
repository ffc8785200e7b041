"""Context-parallel ring attention: ONE long sequence sharded over the ranks of a process group.

The reference has no multi-GPU attention (its kernels see the whole sequence of the local heads);
this module adds the sequence-sharded case on top of the same kernels.  Rank r owns the rows
[r*S/P, (r+1)*S/P) of q, k, v (or, in the "zigzag" layout that balances a causal mask, chunks r and
2P-1-r of 2P).  In step s it attends its queries to the K/V block that started on
rank (r - s) mod P, while that block is already on its way to the next rank: K and V travel as one
buffer, by NCCL send/recv over NVLink, into a second buffer in this GPU's own memory (two buffers per
call, allocated once and used alternately), and no kernel reads another GPU's memory.
Partial results are merged by their log-sum-exp, the same math as the split-KV combine
(csrc/flash_attn/src/flash_fwd_kernel.h:1227-1298).  Masks of a step are expressed with the
`mask_shift` field of the C ABI: shift = (global row of local q row 0) - (global row of block key 0).

Backward runs the ring of K/V blocks a second time; dQ stays local, and what each rank contributes
to the dK/dV of every block stays on that rank in fp32 until one reduce-scatter at the end adds the
contributions up and brings every block's gradient home.  It uses the final (global) LSE and out
of the forward.

With FA_B200_RING_GRAPH=1 the whole forward (and the whole backward) of a call is captured in a CUDA
graph the first time a set of buffers is seen and replayed afterwards.  It is off by default: measured on
8 GPUs the ring is bound by its transfers and its kernels, not by launches (3240 against 3268 TFLOP/s).

The per-block compute is pluggable (`block_ops`) so that the schedule and the merge can be tested on
CPU ranks (gloo) with the oracle standing in for the CUDA kernels.
"""
import ctypes
import os

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------------
class CudaBlockOps:
    """Per-block forward/backward through the C ABI (fa_fwd / fa_bwd with a mask shift)."""

    @staticmethod
    def fwd(q, k, v, scale, window, shift):
        from flash_attention_b200 import _lib
        from flash_attention_b200._lib import FaFwdArgs, check, lib, ptr, tensor3

        B, Sq, H, D = q.shape
        Sk, Hk = k.shape[1], k.shape[2]
        out = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
        a = FaFwdArgs()
        a.q, a.k, a.v, a.out = tensor3(q), tensor3(k), tensor3(v), tensor3(out)
        a.softmax_lse, a.lse_seqlen = ptr(lse), Sq
        a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.heads_k, a.head_dim = B, Sq, Sk, H, Hk, D
        a.dtype = _lib.FA_DTYPE_BF16 if q.dtype == torch.bfloat16 else _lib.FA_DTYPE_FP16
        a.softmax_scale = float(scale)
        a.window_left, a.window_right = int(window[0]), int(window[1])
        a.num_splits = 1
        a.use_mask_shift, a.mask_shift = 1, int(shift)
        stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
        with torch.cuda.device(q.device):
            check(lib().fa_fwd(ctypes.byref(a), stream), "ring block forward")
        return out, lse

    @staticmethod
    def _bwd_args(dout, q, k, v, out, lse, dq, softmax_d, dk_acc, dv_acc, scale, window, shift):
        from flash_attention_b200 import _lib
        from flash_attention_b200._lib import FaBwdArgs, ptr, tensor3

        B, Sq, H, D = q.shape
        Sk, Hk = k.shape[1], k.shape[2]
        a = FaBwdArgs()
        a.q, a.k, a.v, a.out, a.dout, a.dq = (tensor3(x) for x in (q, k, v, out, dout, dq))
        a.softmax_lse, a.lse_seqlen = ptr(lse), lse.stride(1)  # row pitch: lse may be a column range of a wider tensor
        a.softmax_d, a.d_seqlen = ptr(softmax_d), softmax_d.shape[-1]
        a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.heads_k, a.head_dim = B, Sq, Sk, H, Hk, D
        a.dtype = _lib.FA_DTYPE_BF16 if q.dtype == torch.bfloat16 else _lib.FA_DTYPE_FP16
        a.softmax_scale = float(scale)
        a.window_left, a.window_right = int(window[0]), int(window[1])
        a.use_mask_shift, a.mask_shift = 1, int(shift)
        a.accumulate_dkv, a.dk_accum, a.dv_accum = 1, ptr(dk_acc), ptr(dv_acc)
        return a

    @staticmethod
    def bwd(dout, q, k, v, out, lse, dk_acc, dv_acc, scale, window, shift, parts=0):
        """Returns this block's dq (q's dtype); adds the block's dk, dv into the fp32 accumulators.

        parts: 0 the whole backward in one call; (1, 2) two calls on the same buffers, the first of which
        (dot(dO, O) and dQ) does not touch the accumulators yet."""
        from flash_attention_b200._lib import check, lib

        B, Sq, H, D = q.shape
        dq = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
        softmax_d = torch.empty((B, H, (Sq + 127) // 128 * 128), dtype=torch.float32, device=q.device)
        # fp32 workspace of the any-shape kernel (the tensor-core kernels ignore it)
        dq_accum = torch.empty(lib().fa_bwd_workspace_bytes(B, Sq, H, D, 0, 0) // 4, dtype=torch.float32, device=q.device)
        a = CudaBlockOps._bwd_args(dout, q, k, v, out, lse, dq, softmax_d, dk_acc, dv_acc, scale, window, shift)
        a.dq_accum = dq_accum.data_ptr()
        stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
        with torch.cuda.device(q.device):
            for part in (parts if isinstance(parts, tuple) else (parts,)):
                a.parts = part
                check(lib().fa_bwd(ctypes.byref(a), stream), "ring block backward")
        return dq

    @staticmethod
    def merge(out_acc, lse_acc, o, l):
        """In-place LSE merge of the partial (o, l) into the fp32 accumulators (views are fine)."""
        from flash_attention_b200 import _lib
        from flash_attention_b200._lib import check, lib, tensor3

        B, S, H, D = o.shape
        assert out_acc.stride(3) == 1 and o.stride(3) == 1 and lse_acc.stride(2) == 1 and l.stride(2) == 1
        dtype = _lib.FA_DTYPE_BF16 if o.dtype == torch.bfloat16 else _lib.FA_DTYPE_FP16
        stream = ctypes.c_void_p(torch.cuda.current_stream(o.device).cuda_stream)
        ta, tp = tensor3(out_acc), tensor3(o)
        with torch.cuda.device(o.device):
            check(lib().fa_merge_partial(ctypes.byref(ta), lse_acc.data_ptr(), lse_acc.stride(0), lse_acc.stride(1),
                                         ctypes.byref(tp), l.data_ptr(), l.stride(0), l.stride(1), B, S, H, D, dtype, stream),
                  "ring merge")


# ------------------------------------------------------------------------------------------------
def merge_partials(out_a, lse_a, out_b, lse_b):
    """LSE-merge of two partial attention results.  out_*: (B, S, H, D) fp32, lse_*: (B, H, S) fp32
    with +inf or -inf meaning "no visible key".  Returns fp32 (out, lse) with lse = -inf if empty."""
    la = torch.where(torch.isinf(lse_a) & (lse_a > 0), torch.full_like(lse_a, float("-inf")), lse_a)
    lb = torch.where(torch.isinf(lse_b) & (lse_b > 0), torch.full_like(lse_b, float("-inf")), lse_b)
    lse = torch.logaddexp(la, lb)
    wa = torch.exp(la - lse)
    wb = torch.exp(lb - lse)
    wa = torch.where(torch.isnan(wa), torch.zeros_like(wa), wa).transpose(1, 2).unsqueeze(-1)
    wb = torch.where(torch.isnan(wb), torch.zeros_like(wb), wb).transpose(1, 2).unsqueeze(-1)
    return out_a * wa + out_b * wb, lse


def _merge_into(block_ops, out_acc, lse_acc, o, l):
    """out_acc / lse_acc (fp32, -inf = still empty; views allowed) <- merged with the partial (o, l)."""
    fused = getattr(block_ops, "merge", None)
    if fused is not None:
        fused(out_acc, lse_acc, o, l)
    else:
        m_o, m_l = merge_partials(out_acc, lse_acc, o.float(), l)
        out_acc.copy_(m_o)
        lse_acc.copy_(m_l)


def _causal_zigzag_plan(r, src, c):
    """Pure causal mask, zigzag layout, local rows = [early chunk; late chunk] of c rows each.  What
    the queries of rank r see of the K/V that started on rank src is one rectangular call:
      src == r: the local sequence against itself, causally (its two chunks keep their global order);
      src <  r: all local queries against src's early chunk, unmasked;
      src >  r: the late local queries against both of src's chunks, unmasked.
    Returns (q_rows, k_rows, causal) as slices of the local row axis."""
    if src == r:
        return slice(0, 2 * c), slice(0, 2 * c), True
    if src < r:
        return slice(0, 2 * c), slice(0, c), False
    return slice(c, 2 * c), slice(0, 2 * c), False


def _normalize_window(causal, window_size):
    wl, wr = int(window_size[0]), int(window_size[1])
    if causal:
        wr = 0
    return wl, wr


def block_visible(q0, nq, k0, nk, window):
    """Does any (query, key) pair of the two global row ranges satisfy the window rule
    key in [query - wl, query + wr]?  (negative = unbounded)"""
    wl, wr = window
    if wr >= 0 and k0 > q0 + nq - 1 + wr:
        return False
    if wl >= 0 and k0 + nk - 1 < q0 - wl:
        return False
    return True


_KERNELS_ONLY = False


class kernels_only:
    """Measurement aid: inside this context the ring runs its kernels in the same order on this rank's own
    data and exchanges nothing (results are meaningless).  The time of a step in here against a real step
    is the share of the exchange that the kernels do not hide."""

    def __enter__(self):
        global _KERNELS_ONLY
        self.prev, _KERNELS_ONLY = _KERNELS_ONLY, True

    def __exit__(self, *exc):
        global _KERNELS_ONLY
        _KERNELS_ONLY = self.prev


class _P2P:
    """Exchange of one tensor around the ring: send to rank+1, receive from rank-1."""

    def __init__(self, group):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.next = dist.get_global_rank(group, (self.rank + 1) % self.world) if group is not None else (self.rank + 1) % self.world
        self.prev = dist.get_global_rank(group, (self.rank - 1) % self.world) if group is not None else (self.rank - 1) % self.world

    def start(self, send, recv):
        if _KERNELS_ONLY:
            recv.copy_(send)  # same kernels on data of the same kind, nothing crosses NVLink
            return []
        return dist.batch_isend_irecv([dist.P2POp(dist.isend, send, self.next, group=self.group),
                                       dist.P2POp(dist.irecv, recv, self.prev, group=self.group)])

    @staticmethod
    def finish(reqs):
        for r in reqs:
            r.wait()


def ring_steps(layout, world, s_loc, window):
    """Number of ring steps after which no rank can see any key of the block it would receive next
    (the same on every rank).  P for full or causal attention; fewer under a sliding window, e.g. 2 for
    contiguous shards of 4096 rows and window (4096, 0)."""
    last = 0
    for s in range(1, world):
        for r in range(world):
            mine, theirs = layout_chunks(layout, r, world, s_loc), layout_chunks(layout, (r - s) % world, world, s_loc)
            if any(block_visible(qg, qn, kg, kn, window) for qg, qn in mine for kg, kn in theirs):
                last = s
                break
    return last + 1


def layout_chunks(layout, rank, world, s_loc):
    """Global (start, length) of the pieces of the sequence that `rank` holds, in local order.
    "contiguous": rows [rank*s_loc, (rank+1)*s_loc).  "zigzag": the sequence is cut into 2*world
    chunks and rank r holds chunks r and 2*world-1-r, which gives every rank the same amount of
    visible (query, key) area under a causal mask in every step of the ring."""
    if layout == "contiguous":
        return [(rank * s_loc, s_loc)]
    if layout == "zigzag":
        if s_loc % 2:
            raise ValueError("zigzag layout needs an even number of local rows")
        c = s_loc // 2
        return [(rank * c, c), ((2 * world - 1 - rank) * c, c)]
    raise ValueError("unknown layout %r" % (layout,))


def zigzag_shard(x, rank, world, dim=1):
    """The rows of the full sequence `x` that `rank` holds in the zigzag layout."""
    c = x.shape[dim] // (2 * world)
    return torch.cat([x.narrow(dim, rank * c, c), x.narrow(dim, (2 * world - 1 - rank) * c, c)], dim=dim)


def zigzag_unshard(shards, dim=1):
    """Inverse of zigzag_shard over the list of all ranks' shards."""
    world = len(shards)
    c = shards[0].shape[dim] // 2
    chunks = [None] * (2 * world)
    for r, sh in enumerate(shards):
        chunks[r] = sh.narrow(dim, 0, c)
        chunks[2 * world - 1 - r] = sh.narrow(dim, c, c)
    return torch.cat(chunks, dim=dim)


def ring_forward(q, k, v, scale, causal, window_size, group=None, block_ops=CudaBlockOps, layout="contiguous"):
    """Forward of ring attention on this rank's shard. q: (B, S_loc, H, D); k, v: (B, S_loc, Hk, D).
    The global sequence is laid out over the ranks as `layout` says (layout_chunks).  Returns
    (out, lse) with lse fp32 (B, H, S_loc), +inf where a row sees no key."""
    p2p = _P2P(group)
    P, r = p2p.world, p2p.rank
    B, S_loc, H, D = q.shape
    window = _normalize_window(causal, window_size)
    mine = layout_chunks(layout, r, P, S_loc)
    out_acc = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    lse_acc = torch.full((B, H, S_loc), float("-inf"), dtype=torch.float32, device=q.device)
    # one rectangular call per step when the mask is purely causal on zigzag shards of one sequence per batch entry
    fast = layout == "zigzag" and window == (-1, 0) and B == 1
    offs = [sum(n for _, n in mine[:i]) for i in range(len(mine))]
    n_steps = ring_steps(layout, P, S_loc, window)
    # K and V travel as one buffer; two buffers per call, used alternately
    kv = [torch.stack((k, v)), None]
    if n_steps > 1:
        kv[1] = torch.empty_like(kv[0])
    for s in range(n_steps):
        src = (r - s) % P
        cur, nxt = kv[s & 1], kv[(s + 1) & 1]
        reqs = p2p.start(cur, nxt) if s + 1 < n_steps else None
        kc, vc = cur[0], cur[1]
        if fast:
            qs, ks, cz = _causal_zigzag_plan(r, src, S_loc // 2)
            o, l = block_ops.fwd(q[:, qs], kc[:, ks], vc[:, ks], scale, (-1, 0) if cz else (-1, -1), 0)
            _merge_into(block_ops, out_acc[:, qs], lse_acc[:, :, qs], o, l)
        else:
            theirs = layout_chunks(layout, src, P, S_loc)
            for qi, (qg, qn) in enumerate(mine):
                for ki, (kg, kn) in enumerate(theirs):
                    if not block_visible(qg, qn, kg, kn, window):
                        continue
                    qs, ks = slice(offs[qi], offs[qi] + qn), slice(offs[ki], offs[ki] + kn)
                    o, l = block_ops.fwd(q[:, qs], kc[:, ks], vc[:, ks], scale, window, qg - kg)
                    _merge_into(block_ops, out_acc[:, qs], lse_acc[:, :, qs], o, l)
        if reqs is not None:
            p2p.finish(reqs)
    lse = torch.where(torch.isinf(lse_acc) & (lse_acc < 0), torch.full_like(lse_acc, float("inf")), lse_acc)
    return out_acc.to(q.dtype), lse


def _reduce_scatter_sum(parts, group):
    """parts: (P, ...) on every rank; returns the sum over ranks of parts[this rank]."""
    rank = dist.get_rank(group)
    if _KERNELS_ONLY:
        return parts[rank].clone()
    if dist.get_backend(group) == "nccl":
        outp = torch.empty_like(parts[0])
        dist.reduce_scatter_tensor(outp, parts, op=dist.ReduceOp.SUM, group=group)
        return outp
    dist.all_reduce(parts, op=dist.ReduceOp.SUM, group=group)  # backends without reduce-scatter (CPU tests)
    return parts[rank].clone()


def ring_backward(dout, q, k, v, out, lse, scale, causal, window_size, group=None, block_ops=CudaBlockOps,
                  layout="contiguous"):
    """Backward of ring attention.  Returns (dq, dk, dv) of this rank's shards.

    K / V go around the ring a second time.  What a rank contributes to the dK / dV of the block that started on
    rank src stays on that rank, in fp32, in slot src of a (P, ...) buffer, and ONE reduce-scatter at the end adds
    the slots up and brings every block's gradient home.  (Sending fp32 accumulators along with their K / V block
    instead puts twice the bytes of K / V on every hop: measured at 8 ranks, a hop of the accumulators took 0.41 ms
    next to 0.5 ms of kernels per step, and the ring was bound by its transfers.)"""
    p2p = _P2P(group)
    P, r = p2p.world, p2p.rank
    B, S_loc = q.shape[0], q.shape[1]
    window = _normalize_window(causal, window_size)
    mine = layout_chunks(layout, r, P, S_loc)
    offs = [sum(n for _, n in mine[:i]) for i in range(len(mine))]
    fast = layout == "zigzag" and window == (-1, 0) and B == 1
    n_steps = ring_steps(layout, P, S_loc, window)
    kv = [torch.stack((k, v)), None]
    if n_steps > 1:
        kv[1] = torch.empty_like(kv[0])
    # slot src: this rank's share of (dK, dV) of the block that started on rank src
    g = torch.zeros((P,) + tuple(kv[0].shape), dtype=torch.float32, device=k.device)
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    if dout.stride(-1) != 1:
        dout = dout.contiguous()
    for s in range(n_steps):
        src = (r - s) % P
        kv_cur, kv_nxt = kv[s & 1], kv[(s + 1) & 1]
        reqs = p2p.start(kv_cur, kv_nxt) if s + 1 < n_steps else None  # K/V of the next step can already travel
        kc, vc = kv_cur[0], kv_cur[1]
        gk_all, gv_all = g[src, 0], g[src, 1]
        if fast:
            qs, ks, cz = _causal_zigzag_plan(r, src, S_loc // 2)
            # fp32 += 16-bit in one pass over dq
            dq[:, qs].add_(block_ops.bwd(dout[:, qs], q[:, qs], kc[:, ks], vc[:, ks], out[:, qs], lse[:, :, qs], gk_all[:, ks],
                                         gv_all[:, ks], scale, (-1, 0) if cz else (-1, -1), 0))
        else:
            theirs = layout_chunks(layout, src, P, S_loc)
            for qi, (qg, qn) in enumerate(mine):
                for ki, (kg, kn) in enumerate(theirs):
                    if not block_visible(qg, qn, kg, kn, window):
                        continue
                    qs, ks = slice(offs[qi], offs[qi] + qn), slice(offs[ki], offs[ki] + kn)
                    # the accumulators are (B, rows, Hk, D) fp32: a row range of them is itself a dense block per batch entry
                    whole = kn == S_loc or B == 1
                    gk = gk_all[:, ks] if whole else gk_all[:, ks].contiguous()
                    gv = gv_all[:, ks] if whole else gv_all[:, ks].contiguous()
                    dq[:, qs].add_(block_ops.bwd(dout[:, qs], q[:, qs], kc[:, ks], vc[:, ks], out[:, qs], lse[:, :, qs], gk, gv,
                                                 scale, window, qg - kg))
                    if not whole:
                        gk_all[:, ks] = gk
                        gv_all[:, ks] = gv
        if reqs is not None:
            p2p.finish(reqs)
    g_home = _reduce_scatter_sum(g, group) if P > 1 else g[0]
    return dq.to(q.dtype), g_home[0].to(k.dtype), g_home[1].to(v.dtype)


# ------------------------------------------------------------------------------------------------
class _GraphCache:
    """CUDA graphs of whole ring passes, keyed by the buffers and settings they were captured with."""

    def __init__(self, limit=8):
        self.items = {}
        self.limit = limit

    def get(self, key):
        return self.items.get(key)

    def put(self, key, val):
        if len(self.items) >= self.limit:
            self.items.pop(next(iter(self.items)))
        self.items[key] = val


_graphs = _GraphCache()


def release_graphs():
    """Drops every captured graph (and the buffers they own).  Call it before the process group that the graphs'
    communication kernels belong to is destroyed: tearing the communicator down under live graphs can block."""
    if torch.cuda.is_available() and _graphs.items:
        torch.cuda.synchronize()
    _graphs.items.clear()


_graphs_broken = False  # set when a capture failed: later calls launch every step from the host


def _use_graphs(tensors, block_ops):
    if _graphs_broken or block_ops is not CudaBlockOps or not tensors[0].is_cuda:
        return False
    return os.environ.get("FA_B200_RING_GRAPH", "0") == "1"


def _run_captured(kind, fn, inputs, cfg):
    """Runs fn(*inputs) through a CUDA graph captured for exactly these input buffers (addresses, shapes,
    dtypes) and this configuration; captures it on first sight (after one eager run, which also warms up
    NCCL and the kernels' one-time set-up).  Returns fn's outputs, which belong to the graph and are
    overwritten by the next replay."""
    global _graphs_broken
    key = (kind, cfg) + tuple((t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype) for t in inputs)
    hit = _graphs.get(key)
    if hit is None:
        outs = fn(*inputs)  # eager warm-up
        torch.cuda.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                g_outs = fn(*inputs)
        except Exception as e:  # e.g. a communication library that cannot be captured: stay on the host-launched path
            _graphs_broken = True
            import warnings

            warnings.warn("ring attention: CUDA graph capture failed (%s: %s); launching every step from the host" %
                          (type(e).__name__, e))
            return outs
        hit = (graph, g_outs, inputs)  # keep the inputs alive: the graph reads their memory
        _graphs.put(key, hit)
    hit[0].replay()
    return hit[1]


class RingAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, window_size, group, block_ops, layout):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        cfg = (float(softmax_scale), bool(causal), tuple(window_size), id(group), layout)
        if _use_graphs((q, k, v), block_ops):
            qd, kd, vd = q.detach(), k.detach(), v.detach()
            out, lse = _run_captured("fwd", lambda a, b, c: ring_forward(a, b, c, softmax_scale, causal, window_size, group,
                                                                        block_ops, layout), (qd, kd, vd), cfg)
            out, lse = out.clone(), lse.clone()  # the graph's buffers are overwritten by its next replay
        else:
            out, lse = ring_forward(q, k, v, softmax_scale, causal, window_size, group, block_ops, layout)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (softmax_scale, causal, window_size, group, block_ops, layout)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        scale, causal, window_size, group, block_ops, layout = ctx.cfg
        if _use_graphs((q, k, v), block_ops) and dout.stride(-1) == 1:
            cfg = (float(scale), bool(causal), tuple(window_size), id(group), layout)
            # out and lse are fresh tensors of every forward: copy them into buffers that stay with the graph
            key = ("bwd_in", q.data_ptr(), tuple(q.shape))
            held = _graphs.get(key)
            if held is None:
                held = (torch.empty_like(out), torch.empty_like(lse), torch.empty_like(dout))
                _graphs.put(key, held)
            held[0].copy_(out)
            held[1].copy_(lse)
            held[2].copy_(dout)
            dq, dk, dv = _run_captured(
                "bwd", lambda do, a, b, c, o, l: ring_backward(do, a, b, c, o, l, scale, causal, window_size, group, block_ops,
                                                               layout),
                (held[2], q.detach(), k.detach(), v.detach(), held[0], held[1]), cfg)
            dq, dk, dv = dq.clone(), dk.clone(), dv.clone()
        else:
            dq, dk, dv = ring_backward(dout, q, k, v, out, lse, scale, causal, window_size, group, block_ops, layout)
        return dq, dk, dv, None, None, None, None, None, None


def ring_flash_attn_func(q, k, v, softmax_scale=None, causal=False, window_size=(-1, -1), group=None,
                         block_ops=CudaBlockOps, layout="contiguous"):
    """Attention over a sequence that is sharded across the ranks of `group`: contiguous shards in
    rank order, or the load-balanced "zigzag" layout (see layout_chunks, zigzag_shard).  Same
    semantics as flash_attn_func on the gathered sequence (seqlen_q == seqlen_k).

    With FA_B200_RING_GRAPH=1 each pass is replayed from a CUDA graph that is captured the first time a set
    of input buffers is seen."""
    return RingAttnFunc.apply(q, k, v, softmax_scale, causal, tuple(window_size), group, block_ops, layout)
