"""Data-parallel DP training: shard the batch, clip locally, all-reduce the clipped sums.

The reference knows one GPU (example/gpt2/train.py:33) and has no collective.  Samples are
independent, so each rank runs the DP backward on its own B_local samples with
divisor = world * B_local and noise std = noise_multiplier / sqrt(world * B_local), drawing only the
element groups it owns; ONE all-reduce (SUM) of each DP gradient then yields exactly what a single
GPU would compute on the concatenated batch, noise included -- bit-identical noise for any world
size.  Parameters without the `requires_dp` flag carry ordinary local-mean gradients and are
averaged instead.

    reducer = DPGradReducer(model)          # after wrap_with_flashdp_layers, on every rank
    loss.backward(); reducer.finish(); optimizer.step()
"""
import torch
import torch.distributed as dist

from . import runtime


def init_data_parallel(group=None):
    """Read rank / world size from the (already initialised) process group."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    runtime.set_data_parallel(rank, world)
    return rank, world


class DPGradReducer:
    """Bucketed gradient all-reduce that starts as soon as a bucket's gradients exist.

    Buckets follow reverse parameter order (roughly backward order).  When the last gradient of
    a bucket is accumulated, the bucket is packed into a flat buffer and all-reduced
    asynchronously on the communication stream of the backend, so the transfer overlaps the
    rest of the backward pass; `finish()` waits and unpacks.
    """

    def __init__(self, module_or_params, group=None, bucket_bytes=64 << 20, overlap=True):
        params = list(module_or_params.parameters()) if hasattr(module_or_params, "parameters") \
            else list(module_or_params)
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.overlap = overlap
        self.buckets = []          # list of lists of params (same dtype/device)
        cur, cur_bytes, key = [], 0, None
        for p in reversed(self.params):
            k = (p.dtype, p.device)
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
        if overlap and self.world > 1:
            for p in self.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))

    # a non-DP gradient is a local mean: average it; a DP gradient is already divided by the
    # global batch: sum it
    @staticmethod
    def _scale(p, world):
        return 1.0 if getattr(p, "requires_dp", False) else 1.0 / world

    def _launch(self, i):
        bucket = [p for p in self.buckets[i] if p.grad is not None]
        if not bucket:
            return
        parts = []
        for p in bucket:
            sc = self._scale(p, self.world)
            parts.append((p.grad if sc == 1.0 else p.grad * sc).reshape(-1))
        flat = torch.cat(parts)
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._inflight[i] = (work, flat, bucket)

    def _on_grad(self, p):
        i = self._bucket_of[id(p)]
        self._pending[i] -= 1
        if self._pending[i] == 0:
            self._launch(i)

    def finish(self):
        """Wait for every bucket (launching those not yet started) and write the reduced
        gradients back.  Call once per step, after backward and before the optimizer."""
        if self.world > 1:
            for i in range(len(self.buckets)):
                if i not in self._inflight:
                    self._launch(i)
            for i, (work, flat, bucket) in sorted(self._inflight.items()):
                work.wait()
                off = 0
                for p in bucket:
                    n = p.numel()
                    p.grad.copy_(flat[off:off + n].view_as(p.grad))
                    off += n
        self._inflight = {}
        self._pending = [len(b) for b in self.buckets]

    def remove(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []
