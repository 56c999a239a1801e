"""Training-step engine: flat parameter storage, fused Adam, gradient reduction, CUDA-graph replay.

What the reference obtains from ColossalAI's engine (``engine.zero_grad /
backward / step`` with ``HybridAdam`` and DDP, train.py:206-237) is provided
here in one object:

* all parameters live in one flat bf16 buffer (their ``.data`` are views), all
  gradients in one flat bf16 buffer (``.grad`` are views), with fp32 master
  weights and Adam moments beside them; one kernel (csrc/elementwise.cu
  ``adam_k``) updates everything;
* gradients are summed over the whole world (DAP x DP): parameters used on
  DAP-sharded activations need the sum over the DAP group, parameters used in
  replicated computation hold identical gradients on every DAP rank and are
  averaged; the data-parallel mean is folded into the same scale;
* the whole step - forward, loss, recomputation, backward, reduction and
  update - can be captured into one CUDA graph and replayed, which removes the
  host launch cost of the thousands of small kernels of an Evoformer step.
"""
import math

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import param_grad_stream
from ..parallel import core


# Module paths whose parameters act on DAP-sharded activations (each rank sees its shard only, so their gradients are
# summed over the DAP group).  Everything else - embedders, the stacks' closing LayerNorm / projection, structure module,
# heads - runs replicated on the gathered tensors and holds identical gradients on every DAP rank.
DAP_SHARDED_PREFIXES = ("evoformer.blocks.", "extra_msa_stack.blocks.", "template_embedder.template_pair_stack.blocks.",
                        "template_pair_stack.blocks.", "blocks.")


def default_replicated_param_filter(name):
    """``True`` for parameters used in computation that is replicated over the DAP group (their summed gradient is
    divided by the DAP size).  The fast template pair stack scatters its rows between its first and last block, so its
    blocks count as sharded; its closing LayerNorm runs on the gathered tensor and stays replicated."""
    return not name.startswith(DAP_SHARDED_PREFIXES)


def check_device_status(reader=None):
    """Reads the kernels' status word where the host synchronises anyway and raises on EVERY rank when any rank's
    kernels gave up on a bounded wait (a peer that never signalled, a tile that never landed): such a kernel skips the
    data it could not get, so continuing would train or predict on unwritten buffers.  ``reader`` (tests) replaces the
    device read and returns the status list."""
    if reader is None:
        if not torch.cuda.is_available():
            return
        reader = _lib.read_status
    st = list(reader())
    code = int(st[0])
    worst, who = code, core.get_rank()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        t = torch.tensor([code, core.get_rank() if code else -1], device=dev, dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst, who = int(t[0]), int(t[1])
    if worst != 0:
        raise RuntimeError("fastfold_b200: device status %d reported on rank %d (local status %s: code, block x/y/z, detail); "
                           "1 = operand tile never landed, 2 = tensor-core commit missing, 3 = accumulator barrier, "
                           "4 = a peer GPU never raised its flag" % (worst, who, st[:5]))


class FlatAdamTrainer:
    def __init__(self, model, loss_fn, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, use_graph=True,
                 replicated_param_filter=None, grad_reducer=None, grad_sink=True):
        """``loss_fn(model, *inputs) -> scalar loss``.  ``replicated_param_filter(name) -> bool`` marks parameters
        whose computation is replicated (not sharded) over the DAP group.  ``grad_sink=False`` routes every parameter
        gradient through autograd's own accumulation (for comparisons)."""
        self.model = model
        self.loss_fn = loss_fn
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.step_count = 0
        self.use_graph = use_graph and next(model.parameters()).is_cuda
        self.graph = None
        self.static_inputs = None
        self.static_loss = None
        self.graph_fallback = False  # True: a failed capture switches to eager steps instead of raising
        self.aux_getter = None       # callable returning the step's auxiliary outputs (set by the loss function); kept per graph
        self.aux = None
        self._graphs = {}            # graph_key -> (graph, static inputs, static loss, launches)
        self._graph_pool = None
        self.grad_reducer = grad_reducer
        self.launches_per_step = None
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        dev = self.params[0].device
        self.dtype = self.params[0].dtype
        total = sum(p.numel() for p in self.params)
        self.numel = total
        self.flat_w = torch.empty(total, device=dev, dtype=self.dtype)
        # gradients live in the symmetric heap when there is one: the reduction kernel reads and writes peers' copies
        self.grad_heap, self.grad_slot = None, None
        padded = (total + 7) // 8 * 8
        if dev.type == "cuda" and self.dtype == torch.bfloat16 and core.get_world_size() > 1 and grad_reducer is None:
            from ..parallel import symm
            self.grad_heap = symm.get_heap("world")
        if self.grad_heap is not None:
            self.grad_slot = self.grad_heap.slot("flat_grads", padded * 2)
            self.flat_g_padded = self.grad_heap.view(self.grad_slot, (padded,), self.dtype)
            self.flat_g_padded.zero_()
            self.flat_g = self.flat_g_padded[:total]
        else:
            self.flat_g = torch.zeros(total, device=dev, dtype=self.dtype)
        # fp32 gradient sink: weight- and bias-gradient kernels of the fused ops add straight into it (split-K atomics),
        # which removes a zero-fill, a conversion and an accumulate kernel per parameter; folded into flat_g once per step
        self.flat_g32_padded = torch.zeros(padded, device=dev, dtype=torch.float32) if (grad_sink and dev.type == "cuda" and self.dtype == torch.bfloat16) else None
        self.flat_g32 = None if self.flat_g32_padded is None else self.flat_g32_padded[:total]
        if self.grad_heap is None:
            self.flat_g_padded = None
        import os as _os
        self.overlap = _os.environ.get("FASTFOLD_GRAD_OVERLAP", "1") != "0"
        self._overlap_active = False
        self._covered = []
        self._pending = None
        self.bucket_segments = int(_os.environ.get("FASTFOLD_GRAD_BUCKET_SEGMENTS", "12"))
        self._range_of = {}
        self._side = torch.cuda.Stream() if dev.type == "cuda" else None
        if self.grad_heap is not None:
            from ..utils import checkpointing as _ckpt
            _ckpt.POST_BACKWARD_HOOKS[:] = [h for h in _ckpt.POST_BACKWARD_HOOKS if getattr(h, "__self__", None).__class__ is not FlatAdamTrainer]
            _ckpt.POST_BACKWARD_HOOKS.append(self._on_segment_backward)
        self.master = torch.empty(total, device=dev, dtype=torch.float32)
        self.exp_avg = torch.zeros(total, device=dev, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(total, device=dev, dtype=torch.float32)
        self.hp = torch.zeros(4, device=dev, dtype=torch.float32)
        self.hp_host = torch.zeros(4, dtype=torch.float32)
        if dev.type == "cuda":
            self.hp_host = self.hp_host.pin_memory()
        # per-element gradient scale is uniform except for DAP-replicated parameters
        P, D = core.get_dap_size(), core.get_dp_size()
        self.rep_scale = None
        off = 0
        scales = []
        for n, p in params:
            k = p.numel()
            self.flat_w[off:off + k].copy_(p.data.reshape(-1))
            p.data = self.flat_w[off:off + k].view(p.shape)
            p.grad = self.flat_g[off:off + k].view(p.shape)
            if self.flat_g32 is not None:
                from ..ops.gemm import GRAD_SINK_ATTR
                setattr(p, GRAD_SINK_ATTR, self.flat_g32[off:off + k].view(p.shape))
            rep = bool(replicated_param_filter(n)) if replicated_param_filter else False
            scales.append((off, k, rep))
            self._range_of[id(p)] = (off, off + k)
            off += k
        self.master.copy_(self.flat_w.float())
        self.base_gscale = 1.0 / D
        if P > 1 and any(r for _, _, r in scales):
            self.rep_scale = torch.ones(total, device=dev, dtype=self.dtype)
            for o, k, r in scales:
                if r:
                    self.rep_scale[o:o + k] = 1.0 / P

    # ------------------------------------------------------------------
    def _set_hp(self):
        t = self.step_count + 1
        self.hp_host[0] = self.lr
        self.hp_host[1] = 1.0 - self.betas[0] ** t
        self.hp_host[2] = 1.0 - self.betas[1] ** t
        self.hp_host[3] = self.base_gscale
        self.hp.copy_(self.hp_host, non_blocking=True)

    # -- gradient reduction overlapped with backward --------------------------------------------------------------
    # Activation checkpointing runs backward segment by segment (last block first).  As soon as a segment's backward
    # has been enqueued, its slice of the flat gradient buffer is final: a side stream folds the fp32 sink into it and
    # runs the two-shot NVLink all-reduce on just that slice while the main stream goes on with the next segment.
    # What no segment covers (embedders, heads, closing projections) is reduced after backward.  Inside a captured
    # step the side stream is a forked branch of the graph.
    def _segment_range(self, fn):
        blocks = getattr(fn, "__blocks__", None) or [fn]
        lo, hi = None, None
        for b in blocks:
            mod = getattr(b, "func", b)
            mod = getattr(mod, "__self__", mod)
            if not isinstance(mod, torch.nn.Module):
                return None
            for p in mod.parameters():
                r = self._range_of.get(id(p))
                if r is None:
                    continue
                lo = r[0] if lo is None else min(lo, r[0])
                hi = r[1] if hi is None else max(hi, r[1])
        return None if lo is None else (lo, hi)

    def _reduce_range(self, lo, hi):
        """Fold the fp32 sink into ``flat_g[lo:hi]`` and sum that slice over the ranks (``lo``, ``hi`` multiples of 8)."""
        if hi <= lo:
            return
        if self.flat_g32 is not None:
            self.flat_g_padded[lo:hi].add_(self.flat_g32_padded[lo:hi])
        from ..parallel import symm
        _lib.check(symm._libc().ffb_symm_allreduce_bf16(__import__("ctypes").byref(self.grad_heap.ctx), self.grad_slot.index,
                                                        self.grad_slot.offset + lo * 2, hi - lo, 1.0, _lib.stream_ptr()), "symm_allreduce_bf16")

    def _on_segment_backward(self, fn):
        param_grad_stream.join()          # the segment's weight / bias gradients (side stream) are complete from here on
        if not self._overlap_active:
            return
        r = self._segment_range(fn)
        if r is None:
            return
        # elements below the next multiple of 8 belong to the previous segment's slice (reduced later), those up to the
        # next multiple of 8 past the end belong to a segment that is already complete
        lo, hi = (r[0] + 7) // 8 * 8, min((r[1] + 7) // 8 * 8, self.flat_g_padded.numel())
        if hi <= lo:
            return
        # segments arrive back to front and are adjacent in the flat buffer: merge `bucket_segments` of them into one
        # reduction (a fork of the side stream per segment costs more than the small slices are worth)
        if self._pending is not None and self._pending[0] == hi:
            self._pending = (lo, self._pending[1], self._pending[2] + 1)
        else:
            self._flush_pending()
            self._pending = (lo, hi, 1)
        if self._pending[2] >= self.bucket_segments:
            self._flush_pending()

    def _flush_pending(self):
        if self._pending is None:
            return
        lo, hi, _ = self._pending
        self._pending = None
        main = torch.cuda.current_stream()
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            self._reduce_range(lo, hi)
        self._covered.append((lo, hi))

    def _reduce_grads(self):
        if core.get_world_size() > 1:
            if self.grad_reducer is not None:
                self.grad_reducer(self.flat_g)
            elif self.grad_heap is not None and (self._covered or self._pending is not None):
                self._flush_pending()
                torch.cuda.current_stream().wait_stream(self._side)
                pos = 0
                for lo, hi in sorted(self._covered):
                    self._reduce_range(pos, lo)
                    pos = max(pos, hi)
                self._reduce_range(pos, self.flat_g_padded.numel())
            elif self.grad_heap is not None:
                if self.flat_g32 is not None:
                    self.flat_g.add_(self.flat_g32)
                self.grad_heap.all_reduce_(self.grad_slot, self.flat_g_padded.numel())
            else:
                if self.flat_g32 is not None:
                    self.flat_g.add_(self.flat_g32)
                dist.all_reduce(self.flat_g, op=dist.ReduceOp.SUM)
        elif self.flat_g32 is not None:
            self.flat_g.add_(self.flat_g32)
        if self.rep_scale is not None:
            self.flat_g.mul_(self.rep_scale)

    def _adam(self):
        if self.flat_w.is_cuda and self.dtype == torch.bfloat16:
            lib = _lib.get()
            _lib.check(lib.ffb_adam(_lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq), _lib.ptr(self.flat_g),
                                    _lib.ptr(self.flat_w), self.numel, _lib.ptr(self.hp), self.betas[0], self.betas[1], self.eps,
                                    self.wd, _lib.stream_ptr()), "adam")
            return
        lr, bc1, bc2, gs = [float(x) for x in self.hp.tolist()]
        g = self.flat_g.float() * gs
        if self.wd:
            g = g + self.wd * self.master
        self.exp_avg.mul_(self.betas[0]).add_(g, alpha=1 - self.betas[0])
        self.exp_avg_sq.mul_(self.betas[1]).addcmul_(g, g, value=1 - self.betas[1])
        self.master.addcdiv_(self.exp_avg / bc1, (self.exp_avg_sq / bc2).sqrt() + self.eps, value=-lr)
        self.flat_w.copy_(self.master.to(self.dtype))

    def _body(self, inputs):
        self.flat_g.zero_()
        if self.flat_g32 is not None:
            self.flat_g32.zero_()
        loss = self.loss_fn(self.model, *inputs)
        self._covered = []
        self._pending = None
        self._overlap_active = self.overlap and self.grad_heap is not None and self.grad_reducer is None
        param_grad_stream.active = True
        try:
            loss.backward()
        finally:
            self._overlap_active = False
            param_grad_stream.active = False
            param_grad_stream.join()
        self._reduce_grads()
        self._adam()
        return loss.detach()

    # ------------------------------------------------------------------
    def step(self, *inputs, graph_key=None):
        """One optimisation step; returns the (device) loss tensor of this step.

        ``graph_key``: steps whose kernel sequence differs (e.g. the number of recycling iterations of the full model)
        get one captured graph per key, sharing one memory pool; inputs of a key must keep their shapes."""
        self._set_hp()
        if self.use_graph and graph_key is not None:
            if graph_key in self._graphs:
                self.graph, self.static_inputs, self.static_loss, self.launches_per_step, self.aux = self._graphs[graph_key]
            else:
                self.graph = None
        if not self.use_graph:
            n0 = _lib.LAUNCHES[0]
            loss = self._body(inputs)
            self.launches_per_step = _lib.LAUNCHES[0] - n0
            self.step_count += 1
            self.aux = self.aux_getter() if self.aux_getter is not None else None
            return loss
        if self.graph is None and self.graph_fallback:
            try:
                return self._capture_and_replay(inputs, graph_key)
            except Exception as e:      # noqa: BLE001 - e.g. an op that reads a value on the host during capture
                import logging
                logging.getLogger("fastfold_b200").warning("CUDA-graph capture of the training step failed (%s); running eagerly", repr(e)[:200])
                torch.cuda.synchronize()
                self.use_graph = False
                self.graph = None
                return self.step(*inputs)
        return self._capture_and_replay(inputs, graph_key)

    def _capture_and_replay(self, inputs, graph_key):
        if self.graph is None:
            self.static_inputs = [x.clone() if isinstance(x, torch.Tensor) else x for x in inputs]
            # warm-up on a side stream (allocator, cuBLAS handles, NCCL channels), then capture
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    self._body(self.static_inputs)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            # the two warm-up passes are real optimisation steps and are counted as such
            self.graph = torch.cuda.CUDAGraph()
            n0 = _lib.LAUNCHES[0]
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(self.graph, pool=self._graph_pool):
                self.static_loss = self._body(self.static_inputs)
            self.launches_per_step = _lib.LAUNCHES[0] - n0
            self.step_count += 2
            self._set_hp()
            self.aux = self.aux_getter() if self.aux_getter is not None else None
            if graph_key is not None:
                self._graphs[graph_key] = (self.graph, self.static_inputs, self.static_loss, self.launches_per_step, self.aux)
        else:
            for dst, src in zip(self.static_inputs, inputs):
                if isinstance(dst, torch.Tensor) and dst.data_ptr() != src.data_ptr():
                    dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.step_count += 1
        return self.static_loss

    def check_status(self, reader=None):
        """Raise (on all ranks) if any rank's kernels recorded a failed wait since the last check; synchronises."""
        check_device_status(reader)

    def state_dict(self):
        return {"step": self.step_count, "master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "lr": self.lr, "names": self.names}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.lr = sd.get("lr", self.lr)
        self.flat_w.copy_(self.master.to(self.dtype))
