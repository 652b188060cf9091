"""Data-parallel DP training: shard the batch, clip locally, all-reduce the clipped sums.

The reference knows one GPU (example/gpt2/train.py:33) and has no collective.  Samples are
independent, so each rank runs the DP backward on its own B_local samples with
divisor = world * B_local and noise std = noise_multiplier / sqrt(world * B_local), drawing only the
element groups it owns; ONE all-reduce (SUM) of each DP gradient then yields exactly what a single
GPU would compute on the concatenated batch, noise included: element i's noise is the same draw
z_i(seed, param_id, step) for any world size, added by exactly one rank (the gradient it is added to
is an fp32 sum whose association differs with the sharding, so whole results agree to rounding, not
bit for bit).  Parameters without the `requires_dp` flag carry ordinary local-mean gradients and are
averaged instead.

    reducer = DPGradReducer(model)          # after wrap_with_flashdp_layers, on every rank
    loss.backward(); reducer.finish(); optimizer.step(); reducer.zero_grad()

With `grad_as_bucket_view=True` every `p.grad` is a view into its bucket's flat buffer: autograd
accumulates into the bucket in place, the all-reduce runs on the buffer itself and nothing is
packed or unpacked.  With gradient accumulation (runtime.accumulate) pass `sync=False` to
`finish()` on all but the last micro-step.
"""
import weakref

import torch
import torch.distributed as dist
from torch.utils.weak import WeakIdKeyDictionary

from . import runtime


# DP parameter -> weak reference to the reducer whose bucket slices it may be written into.  Kept
# here rather than as an attribute of the parameter, so that parameters stay picklable.
_direct = WeakIdKeyDictionary()     # keyed by identity: tensors do not compare with ==


def direct_reducer(param):
    """The live DPGradReducer offering bucket slices for `param`, or None."""
    ref = _direct.get(param)
    return ref() if ref is not None else None


def init_data_parallel(group=None):
    """Read rank / world size from the (already initialised) process group and give every rank
    rank 0's noise seed (the ranks draw disjoint parts of ONE noise tensor, which is reproducible
    across world sizes only under a common key)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    runtime.set_data_parallel(rank, world)
    if world > 1:
        box = [runtime.get_seed()]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        runtime.manual_seed(box[0])
    return rank, world


class DPGradReducer:
    """Bucketed gradient all-reduce that starts as soon as a bucket's gradients exist.

    Buckets follow reverse parameter order (roughly backward order).  When the last gradient of
    a bucket is accumulated, the bucket is packed into a flat buffer and all-reduced
    asynchronously on the communication stream of the backend, so the transfer overlaps the
    rest of the backward pass; `finish()` waits and unpacks.  With `grad_as_bucket_view` the
    gradients live in the flat buffers from the start (buckets then hold either DP tensors, which
    are summed, or ordinary ones, which are averaged) and packing/unpacking disappears.
    """

    def __init__(self, module_or_params, group=None, bucket_bytes=64 << 20, overlap=True,
                 grad_as_bucket_view=False, direct_write=True):
        params = list(module_or_params.parameters()) if hasattr(module_or_params, "parameters") \
            else list(module_or_params)
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.overlap = overlap
        self.as_view = grad_as_bucket_view
        self.buckets = []          # list of lists of params (same dtype/device; with views also same scale)
        cur, cur_bytes, key = [], 0, None
        for p in reversed(self.params):
            k = (p.dtype, p.device, self._scale(p, self.world) if self.as_view else None)
            nbytes = p.numel() * p.element_size()
            if cur and (k != key or cur_bytes + nbytes > bucket_bytes):
                self.buckets.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            key = k
        if cur:
            self.buckets.append(cur)
        self._bucket_of = {id(p): i for i, b in enumerate(self.buckets) for p in b}
        self._pending = [len(b) for b in self.buckets]
        self._inflight = {}
        self._hooks = []
        self._sync = True
        self._reserve_prev = None
        self._claimed, self._counted = set(), set()
        self._flat, self._views = [], {}
        if self.as_view:
            for b in self.buckets:
                # every slice starts on a 64-byte boundary (the kernels want 16-byte-aligned outputs)
                quantum = 64 // b[0].element_size()
                starts, off = [], 0
                for p in b:
                    starts.append(off)
                    off += (p.numel() + quantum - 1) // quantum * quantum
                flat = torch.zeros(off, dtype=b[0].dtype, device=b[0].device)
                for p, st in zip(b, starts):
                    self._views[id(p)] = flat[st:st + p.numel()].view_as(p)
                self._flat.append(flat)
            self._attach_views()
            if direct_write:
                # DP layers may write a weight gradient straight into its bucket slice (claim_direct)
                for p in self.params:
                    if getattr(p, "requires_dp", False):
                        _direct[p] = weakref.ref(self)
        if overlap and self.world > 1:
            for p in self.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))

    def _attach_views(self):
        for i in range(len(self.buckets)):
            self._attach_views_of(i)

    def zero_grad(self):
        """Zero the gradients while keeping them views of the buckets (an optimizer's
        zero_grad(set_to_none=True) would detach them; the next finish() re-attaches by copy)."""
        if self.as_view:
            for flat in self._flat:
                flat.zero_()
            self._attach_views()
            self._claimed.clear()
        else:
            for p in self.params:
                p.grad = None

    def claim_direct(self, p):
        """The bucket slice of `p` if the coming gradient may overwrite it, else None: the first
        gradient after zero_grad() (or after the gradient was set to None) overwrites, later ones
        are returned to autograd, which adds them to the slice -- torch's accumulation semantics.
        Assumes a DP weight takes part in one layer call per backward pass (build the reducer with
        direct_write=False for a model that shares a DP weight between layers)."""
        if not self.as_view or id(p) not in self._views:
            return None
        if id(p) in self._claimed and p.grad is not None:
            return None
        self._claimed.add(id(p))
        p.grad = self._views[id(p)]
        return p.grad

    def direct_written(self, p):
        if self._hooks:
            self._on_grad(p)

    def set_sync(self, sync: bool):
        """sync=False: the coming backward is an accumulation micro-step -- gradients pile up
        locally and no collective starts.  Set it back to True before the last micro-step."""
        self._sync = bool(sync)

    # a non-DP gradient is a local mean: average it; a DP gradient is already divided by the
    # global batch: sum it
    @staticmethod
    def _scale(p, world):
        return 1.0 if getattr(p, "requires_dp", False) else 1.0 / world

    def _launch(self, i):
        if self.as_view:
            self._attach_views_of(i)
            flat, bucket = self._flat[i], self.buckets[i]
            sc = self._scale(bucket[0], self.world)
            if sc != 1.0:
                flat.mul_(sc)
        else:
            bucket = [p for p in self.buckets[i] if p.grad is not None]
            if not bucket:
                return
            parts = []
            for p in bucket:
                sc = self._scale(p, self.world)
                parts.append((p.grad if sc == 1.0 else p.grad * sc).reshape(-1))
            flat = torch.cat(parts)
        if not self._inflight and self.world > 1 and flat.is_cuda and runtime.reserve_sms() > 0:
            # from the first collective of this step until finish(): the library's GEMM grids leave a
            # few SMs free for the all-reduce kernels (off unless FDP_DP_RESERVE_SMS asks for it)
            self._reserve_prev = self._set_reserve(runtime.reserve_sms())
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._inflight[i] = (work, flat, bucket)

    @staticmethod
    def _set_reserve(n):
        from . import _lib
        return _lib.load().fdp_set_sm_reserve(int(n))

    def _attach_views_of(self, i):
        """Make every gradient of bucket i a view of its flat buffer; a gradient that autograd
        allocated itself (after a zero_grad(set_to_none=True)) is copied in first, a missing one
        counts as zero."""
        for p in self.buckets[i]:
            v = self._views[id(p)]
            if p.grad is None:
                v.zero_()              # nothing arrived since the gradient was reset
            elif p.grad.data_ptr() != v.data_ptr():
                v.copy_(p.grad)
            p.grad = v

    def _on_grad(self, p):
        if not self._sync or id(p) in self._counted:
            return
        self._counted.add(id(p))
        i = self._bucket_of[id(p)]
        self._pending[i] -= 1
        if self._pending[i] == 0:
            self._launch(i)

    def finish(self, sync=None):
        """Wait for every bucket (launching those not yet started) and write the reduced
        gradients back.  Call once per optimizer step, after the (last) backward and before the
        optimizer; `sync=False` skips the collective (an accumulation micro-step)."""
        if sync is None:
            sync = self._sync
        if self.world > 1 and sync:
            for i in range(len(self.buckets)):
                if i not in self._inflight:
                    self._launch(i)
            for i, (work, flat, bucket) in sorted(self._inflight.items()):
                work.wait()
                if self.as_view:
                    continue
                off = 0
                for p in bucket:
                    n = p.numel()
                    p.grad.copy_(flat[off:off + n].view_as(p.grad))
                    off += n
        if self._reserve_prev is not None:
            self._set_reserve(self._reserve_prev)
            self._reserve_prev = None
        if self.params and self.params[0].is_cuda:
            runtime.check_device_status(self.params[0].device.index)
        self._inflight = {}
        self._pending = [len(b) for b in self.buckets]
        self._counted.clear()

    def remove(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []
        for p in self.params:
            if direct_reducer(p) is self:
                del _direct[p]
