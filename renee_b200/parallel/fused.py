"""Collectives fused into the compute kernels over NVLink peer memory.

:class:`PeerCollectives` keeps the interface of :class:`~renee_b200.parallel.collectives.TorchCollectives`
but moves the per-step data path off NCCL:

==========================  ==================================================================
exchange                    realisation
==========================  ==================================================================
all-gather of embeddings    the pooling/dropout kernel of each rank stores its fp16 rows straight
                            into EVERY rank's ``X`` buffer and raises a flag; the logits GEMM's
                            producer warp waits for the flags before its first TMA load
reduce-scatter of ``dX``    the dX GEMM accumulates into this rank's partial buffer; its last CTA
                            raises a flag on every rank; a pull kernel sums this rank's rows over
                            all partials (and applies the dropout backward)
encoder gradients +         sharded optimizer: each rank sums its 1/G slice of the flat gradient over
AdamW                       all ranks (NVLS ``multimem.ld_reduce`` or peer loads), reports non-finite
                            values to everyone, applies AdamW to its slice of the fp32 masters and
                            stores the new 16-bit weights into every rank's compute copy
                            (``multimem.st`` or peer stores); a non-sharded two-shot all-reduce
                            kernel is kept as well
==========================  ==================================================================

Buffers that peers write or read (``X``, the ``dX`` partials) are double-buffered by step parity;
flags carry the step number read from a device-resident counter, so the launch sequence is identical
every step and can be replayed from a CUDA graph (two graphs, one per parity).  By default the
buffers are plain ``cudaMalloc`` allocations mapped into the other ranks with CUDA IPC — peer-to-peer
only, no NVLink multicast object is ever bound, so a rank that dies cannot fault the survivors' GPUs
through one.  With ``use_nvls=True`` (or ``RENEE_B200_NVLS=1``; meant for benchmark runs) they come from
``torch.distributed._symmetric_memory`` and the gradient reduction and parameter push go through the
switch's multicast mapping (``multimem``).  NCCL remains for bootstrap, evaluation merges and scalars.
No TMA multicast is used anywhere.

Safety of the buffer reuse (rank r at step n+2 may overwrite what rank q read at step n): r can only
reach step n+2's overwrite after finishing its own pull of step n+1, which waited for q's step-(n+1)
dX flag, which q raised after its step-n pull in stream order.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..utils import guard
from ..utils.sharding import batch_row_range
from .collectives import TorchCollectives
from .dist import DistContext

# word offsets of the flag classes inside the symmetric flag array (16 words each)
F_AG, F_RS, F_ARA, F_ARB, F_FOUND, F_ARC, F_EV = 0, 16, 32, 48, 64, 80, 96
FLAG_WORDS = 128


class PeerCollectives(TorchCollectives):
    graph_safe = True

    def __init__(self, ctx: DistContext, group=None, shard_optimizer: bool = True, use_nvls: bool | None = None):
        super().__init__(ctx)
        self.shard_optimizer = shard_optimizer
        # NVLS (multimem loads/stores through the NVSwitch multicast mapping) for the gradient reduction
        # and the parameter push is OPT-IN (use_nvls=True or RENEE_B200_NVLS=1): a crash, an OOM kill or a
        # PeerFailure exit of one rank while its memory is bound to a multicast object can raise NVLink
        # faults on the other ranks' GPUs, and the bounded flag waits do not cover a multimem access whose
        # member has gone.  The default stays on plain peer loads/stores over CUDA IPC mappings.
        self.use_nvls = (os.environ.get("RENEE_B200_NVLS", "0") == "1") if use_nvls is None else bool(use_nvls)
        self._mc_grad = 0
        self._mc_p16 = 0
        self.p16 = None
        self.gsum = None
        if ctx.device.type != "cuda":
            raise RuntimeError("PeerCollectives needs CUDA devices")
        if self.G > 16:
            raise RuntimeError("at most 16 peers")
        self.group = group if group is not None else dist.group.WORLD
        self._handles = []
        self._ready = False
        self.grad = None
        self.host_step = 0
        self._comm_stream = None

    # ------------------------------------------------------------------ allocation
    def _symm(self, numel: int, dtype, name: str = "symmetric"):
        """``(local tensor, [device address of the same buffer on every rank])``."""
        if not self.use_nvls:
            return self._ipc(numel, dtype, name)
        import torch.distributed._symmetric_memory as symm_mem
        whole = []

        def alloc(n, dt):
            whole.append(symm_mem.empty(n, dtype=dt, device=self.ctx.device))
            return whole[0]

        # in guard mode the payload sits one band into the allocation on every rank: shift the peer and
        # multicast addresses by the same amount
        t = guard.from_allocator(alloc, numel, dtype, name=f"{name}{len(self._handles)}")
        off = guard.payload_offset_bytes()
        hdl = symm_mem.rendezvous(whole[0], self.group)
        self._handles.append(hdl)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0) if self.use_nvls else 0
        self._last_multicast = mc + off if mc else 0
        return t, [int(p) + off for p in hdl.buffer_ptrs]

    def _ipc(self, numel: int, dtype, name: str):
        """Peer-mapped only: own ``cudaMalloc`` block, handles exchanged over the process group, every
        peer's block opened with ``cudaIpcOpenMemHandle``.  Collective (every rank calls it in the same order)."""
        from ..ops import cuda as cu
        whole = []

        def alloc(n, dt):
            whole.append(cu.ipc_alloc(n, dt, self.ctx.device))
            return whole[0]

        t = guard.from_allocator(alloc, numel, dtype, name=f"{name}{len(self._handles)}")
        off = guard.payload_offset_bytes()
        handles = [None] * self.G
        dist.all_gather_object(handles, cu.ipc_export(whole[0]), group=self.group)
        ptrs = [whole[0].data_ptr() if r == self.rank else cu.ipc_open(handles[r], self.ctx.device)
                for r in range(self.G)]
        self._handles.append((whole[0], ptrs))
        self._last_multicast = 0
        return t, [p + off for p in ptrs]

    def setup(self, B_max: int, D: int) -> None:
        from ..ops import cuda as cu
        if self._ready:
            return
        dev = self.ctx.device
        rows = B_max + self.G
        self.D = D
        self.flags, flag_ptrs = self._symm(FLAG_WORDS, torch.int32)
        self.flags.zero_()
        self.X, self.dXp, self._x_ptrs, self._dx_ptrs = [], [], [], []
        for _ in range(2):
            x, xp = self._symm(rows * D, torch.float16)
            d, dp = self._symm(rows * D, torch.float32)
            x.zero_(); d.zero_()
            self.X.append(x.view(rows, D)); self.dXp.append(d.view(rows, D))
            self._x_ptrs.append(cu.ptr_array(xp)); self._dx_ptrs.append(cu.ptr_array(dp))
        self._flag_ptrs = cu.ptr_array(flag_ptrs)
        self.step = torch.zeros(1, dtype=torch.int32, device=dev)
        self.counters = torch.zeros(64, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._ready = True

    def alloc_grad(self, numel: int, dtype) -> torch.Tensor:
        """Flat encoder-gradient buffer in symmetric memory (peers read and write it)."""
        from ..ops import cuda as cu
        n = (numel + 1023) // 1024 * 1024
        self.grad, gp = self._symm(n, dtype)
        self._mc_grad = self._last_multicast
        self.grad.zero_()
        self._grad_ptrs = cu.ptr_array(gp)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        return self.grad

    def alloc_p16(self, numel: int, dtype) -> torch.Tensor:
        """Low-precision compute copy of the encoder parameters in symmetric memory: with the sharded
        optimizer every rank stores its freshly updated slice into every rank's copy."""
        from ..ops import cuda as cu
        n = (numel + 1023) // 1024 * 1024
        self.p16, pp = self._symm(n, dtype)
        self._mc_p16 = self._last_multicast
        self.p16.zero_()
        self._p16_ptrs = cu.ptr_array(pp)
        per = ((numel // 8) + self.G - 1) // self.G * 8
        self.gsum = guard.zeros(per + 8, dtype=torch.float32, device=self.ctx.device, name="optimizer.gsum")
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        return self.p16

    def slice_range(self, numel: int, rank: int) -> tuple[int, int]:
        n_vec = numel // 8
        per = (n_vec + self.G - 1) // self.G
        return min(n_vec, per * rank) * 8, min(n_vec, per * (rank + 1)) * 8

    def _sharded(self, enc) -> bool:
        return (self.shard_optimizer and self.p16 is not None and self.grad is not None
                and enc.g.data_ptr() == self.grad.data_ptr() and enc.p16.data_ptr() == self.p16.data_ptr())

    # ------------------------------------------------------------------ sharded optimizer, overlapped with backward
    def _buckets(self, enc):
        """Splits the flat gradient buffer into buckets that become final at successive points of the backward pass
        and gives every rank 1/G of EACH bucket (so every rank has work for every bucket, also for the last and
        largest one, the embeddings).  Stage ``s`` = 1 .. n_layers is reached when layer ``n_layers - s`` is done,
        stage ``n_layers + 1`` at the end of the pass (embeddings, bottleneck, and the no-decay tail of the buffer:
        biases and LayerNorm parameters of all layers).  Returns ``[(stage, v0, v1, g0)]`` for this rank: vector
        (8-element) ranges of the flat buffer and the offset of their sums in ``gsum``."""
        key = (id(enc), enc.numel)
        if getattr(self, "_bucket_key", None) == key:
            return self._bucket_plan
        L = enc.cfg.n_layers
        start = [enc.slots[f"transformer.layer.{l}.attention.q_lin.weight"].offset for l in range(L)]
        last = enc.slots[f"transformer.layer.{L - 1}.ffn.lin2.weight"]
        end = start[1:] + [(last.offset + last.numel + 127) // 128 * 128]   # a layer's matrices are contiguous
        ranges = [(L - l, start[l], end[l]) for l in reversed(range(L))]            # (stage, lo, hi) in elements
        ranges += [(L + 1, 0, start[0]), (L + 1, end[-1], enc.numel // 8 * 8)]
        plan, g0 = [], 0
        for stage, lo, hi in ranges:
            n_vec = (hi - lo) // 8
            per = (n_vec + self.G - 1) // self.G
            a = lo // 8 + min(n_vec, per * self.rank)
            b = lo // 8 + min(n_vec, per * (self.rank + 1))
            if b > a:
                plan.append((stage, a, b, g0))
                g0 += b - a
        need = g0 * 8
        if self.gsum is None or self.gsum.numel() < need:
            self.gsum = guard.zeros(need + 8, dtype=torch.float32, device=self.ctx.device, name="optimizer.gsum")
        self._bucket_plan, self._bucket_key = plan, key
        self._bucket_ranges = ranges
        self._n_stages = L + 1
        return plan

    def owned_ranges(self, enc, rank: int):
        """Element ranges of the flat buffer whose master weights rank ``rank`` keeps up to date."""
        self._buckets(enc)
        out = []
        for _, lo, hi in self._bucket_ranges:
            n_vec = (hi - lo) // 8
            per = (n_vec + self.G - 1) // self.G
            a, b = lo + min(n_vec, per * rank) * 8, lo + min(n_vec, per * (rank + 1)) * 8
            if b > a:
                out.append((a, b))
        return out

    def backward_begin(self, enc) -> None:
        """Called before the encoder backward: the reduction of finished buckets runs on a second stream."""
        # Opt-in (RENEE_B200_RS_OVERLAP=1).  Measured on B200s at the 131 K-label config, overlapped / in one piece after
        # the pass: 2.42 / 2.31 ms per step on 2 GPUs, 1.75 / 1.66 on 4 (and 5.53 / 5.49 at 1.3 M labels on 2): the
        # per-layer signal kernels and the bucket kernels' share of the SMs cost the short backward pass of a rank
        # more than the hidden transfer (at most 133 MB of 16-bit gradients over NVLink, about 0.15 ms) saves.
        if not self._sharded(enc) or os.environ.get("RENEE_B200_RS_OVERLAP", "0") != "1":
            return
        self._buckets(enc)
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=self.ctx.device)
        self._stage = 0

    def on_layer_done(self, enc, layer: int) -> None:
        """Gradient of ``layer`` (``-1``: the embeddings, i.e. the end of the pass) is final on this rank: tell the
        peers, and reduce this rank's part of the bucket as soon as every peer has told the same."""
        from ..ops import cuda as cu
        if not self._sharded(enc) or self._comm_stream is None:
            return
        L = enc.cfg.n_layers
        stage = L - layer if layer >= 0 else L + 1
        self._stage = stage
        last = stage == L + 1
        main = torch.cuda.current_stream()
        # progress flag: step * 32 + stage (monotone within a step and from step to step)
        cu.signal(self._flag_ptrs, self.G, F_ARA, self.rank, self.step, 32, stage)
        side = self._comm_stream
        side.wait_stream(main)
        with torch.cuda.stream(side):
            mine = [b for b in self._bucket_plan if b[0] == stage]
            blocks = cu.sm_count(self.ctx.device) * 2 if last else 32      # few CTAs while the backward GEMMs run
            for i, (_, a, b, g0) in enumerate(mine):
                final = last and i == len(mine) - 1
                cu.grad_reduce_scatter_range(enc.g.dtype, self._grad_ptrs, a, b, self.G, self.rank, self.flags[F_ARA:],
                                             self.step, 32, stage, self.gsum[g0 * 8:], self._flag_ptrs,
                                             F_ARB if final else -1, F_FOUND, self.counters[48:], blocks,
                                             mc_grads=self._mc_grad)
            if last and not mine:
                # nothing of the last bucket is this rank's: still tell the peers that its reductions are done
                cu.signal(self._flag_ptrs, self.G, F_ARB, self.rank, self.step)
        if last:
            main.wait_stream(side)

    def optimizer_step(self, enc, hp, beta1, beta2, eps, wd) -> None:
        """Sharded AdamW: reduce-scatter of the gradients, AdamW on this rank's part of the masters, push of
        the updated 16-bit values into every rank's compute copy.  The found-inf decision is global because
        the update only starts after every rank's reductions (and their non-finite reports) have landed.  When
        the trainer drove ``backward_begin`` / ``on_layer_done`` the reductions already ran, bucket by bucket, under
        the backward pass; otherwise they run here in one piece."""
        from ..ops import cuda as cu
        if not self._sharded(enc):
            return super().optimizer_step(enc, hp, beta1, beta2, eps, wd)
        plan = self._buckets(enc)
        sms = cu.sm_count(self.ctx.device)
        if getattr(self, "_stage", 0) != self._n_stages:
            # not overlapped (eager callers, tests): every bucket now, all flags at their final value
            cu.signal(self._flag_ptrs, self.G, F_ARA, self.rank, self.step, 32, self._n_stages)
            for i, (_, a, b, g0) in enumerate(plan):
                cu.grad_reduce_scatter_range(enc.g.dtype, self._grad_ptrs, a, b, self.G, self.rank, self.flags[F_ARA:],
                                             self.step, 32, self._n_stages, self.gsum[g0 * 8:], self._flag_ptrs,
                                             F_ARB if i == len(plan) - 1 else -1, F_FOUND, self.counters[48:], sms * 2,
                                             mc_grads=self._mc_grad)
            if not plan:
                cu.signal(self._flag_ptrs, self.G, F_ARB, self.rank, self.step)
        self._stage = 0
        cu.wait_flags(self.flags[F_ARB:], self.G, self.step, 1, 0, self.flags[F_FOUND:], hp.buf)
        cu.adamw_ranges_push(enc.p16.dtype, enc.p32, enc.m, enc.v, self.gsum, self._p16_ptrs,
                             [(a, b, g0) for _, a, b, g0 in plan], enc.n_decay, self.G, self.rank, hp.buf, beta1, beta2,
                             eps, wd, 1.0 / self.G, self._flag_ptrs, F_ARC, self.step, self.counters[52:], sms * 2,
                             mc_p16=self._mc_p16)
        cu.wait_flags(self.flags[F_ARC:], self.G, self.step, 1, 0, None, None)

    def sync_master(self, enc) -> None:
        """Collective: after it, every rank holds the complete fp32 master weights (each rank owns the
        up-to-date values of its slice only).  Called before state dicts are taken."""
        if not self._sharded(enc):
            return
        for r in range(self.G):
            for lo, hi in self.owned_ranges(enc, r):
                dist.broadcast(enc.p32[lo:hi], src=r, group=self.group)

    # ------------------------------------------------------------------ per-step protocol
    @property
    def parity(self) -> int:
        return self.host_step & 1

    def host_begin(self) -> None:
        """Host side of a new step: flips the buffer parity.  Must be called once per step, whether the
        device work is then launched eagerly or replayed from a graph."""
        self.host_step += 1

    def device_begin(self) -> None:
        """Device side of a new step: advances the step counter the flag tags derive from."""
        from ..ops import cuda as cu
        cu.step_inc(self.step)

    def embeddings_to_X(self, emb, B, p, rng, stream_id, bufs):
        from ..ops import cuda as cu
        s, e = batch_row_range(B, self.G, self.rank)
        cu.ag_push(emb, p, rng, stream_id, self._x_ptrs[self.parity], s, self._flag_ptrs, F_AG, self.rank, self.G,
                   self.step, self.counters)
        X = self.X[self.parity][:B]
        return X, (self.flags[F_AG:], self.G, self.step)

    def dx_buffer(self, B, bufs):
        return self.dXp[self.parity][:B], (self.counters[32:], self._flag_ptrs, self.G, F_RS + self.rank, self.step)

    def dx_to_local(self, dX, B, p, rng, stream_id, bufs):
        from ..ops import cuda as cu
        s, e = batch_row_range(B, self.G, self.rank)
        de = bufs["de"][: e - s]
        cu.rs_pull(self._dx_ptrs[self.parity], self.G, s, e - s, self.D, de, self.flags[F_RS:], self.step, p, rng, stream_id)
        return de

    # ------------------------------------------------------------------ prediction: cross-rank top-k merge
    def merge_topk(self, vals: torch.Tensor, idxs: torch.Tensor, k: int):
        """``vals/idxs [n, k]`` per rank (global label ids) → global top-k on every rank, over peer memory: every rank
        stores its candidates (values and ids packed in one ``[n, 2k]`` block) into slot ``rank`` of every rank's
        buffer and raises a flag; after all flags one selection kernel picks the k best of the ``G k`` candidates
        of a row.  Buffers alternate by call parity (a rank can be at most one call ahead of a peer)."""
        from ..ops import cuda as cu
        if self.G == 1 or not vals.is_cuda:
            return super().merge_topk(vals, idxs, k)
        n, kk = vals.shape
        width = (2 * kk + 3) // 4 * 4                                   # floats per row, a multiple of 16 bytes
        need = n * width
        if getattr(self, "_ev_cap", 0) < need:
            cap = max(need, 256 * 256)
            self._ev_buf, self._ev_ptrs = [], []
            for _ in range(2):
                t, ptrs = self._symm(self.G * cap, torch.float32, name="eval.topk")
                self._ev_buf.append(t)
                self._ev_ptrs.append(cu.ptr_array(ptrs))
            self._ev_cap = cap
            self._ev_step = torch.zeros(1, dtype=torch.int32, device=self.ctx.device)
            self._ev_calls = 0
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        self._ev_calls += 1
        par = self._ev_calls & 1
        pack = torch.zeros(n, width, dtype=torch.float32, device=vals.device)
        pack[:, :kk] = vals.float()
        pack[:, kk:2 * kk] = idxs.to(torch.int32).view(torch.float32)
        cu.step_inc(self._ev_step)
        cu.peer_gather(pack, self._ev_ptrs[par], self.rank * self._ev_cap * 4, self._flag_ptrs, F_EV, self.rank, self.G,
                       self._ev_step, self.counters[16:])
        cu.wait_flags(self.flags[F_EV:], self.G, self._ev_step, 1, 0, None, None)
        got = self._ev_buf[par].view(self.G, self._ev_cap)[:, :need].view(self.G, n, width)
        cv = got[:, :, :kk].permute(1, 0, 2).reshape(n, self.G * kk).contiguous()
        ci = got[:, :, kk:2 * kk].permute(1, 0, 2).reshape(n, self.G * kk).contiguous().view(torch.int32)
        k_eff = min(k, self.G * kk)
        ov = torch.empty(n, k_eff, dtype=torch.float32, device=vals.device)
        op = torch.empty(n, k_eff, dtype=torch.int32, device=vals.device)
        cu.topk_rows(cv, self.G * kk, k_eff, 0, ov, op)
        v, order = torch.sort(ov, dim=1, descending=True)
        return v, torch.gather(torch.gather(ci, 1, op.long()), 1, order).long()

    def allreduce_grads(self, g: torch.Tensor, hp) -> float:
        from ..ops import cuda as cu
        if self.grad is None or g.data_ptr() != self.grad.data_ptr() or g.dtype == torch.float32:
            return super().allreduce_grads(g, hp)
        n = g.numel() // 8 * 8
        cu.signal(self._flag_ptrs, self.G, F_ARA, self.rank, self.step)
        cu.grad_allreduce(g.dtype, self._grad_ptrs, 0, n, self.G, self.rank, self.flags[F_ARA:], self._flag_ptrs, F_ARB,
                          F_FOUND, self.step, 1, 0, self.counters[48:], cu.sm_count(self.ctx.device) * 2)
        cu.wait_flags(self.flags[F_ARB:], self.G, self.step, 1, 0, self.flags[F_FOUND:], hp.buf)
        return 1.0 / self.G
