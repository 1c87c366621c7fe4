"""Batch-sharded data parallelism for the recurrent layers: one process per GPU.

Every sequence of a batch is independent and LayerNorm statistics are per row, so a layer
shards on the batch axis with no exchange in the forward or backward pass; the only
collective is the sum of the parameter gradients (kernel, recurrent kernel, biases,
LayerNorm gains) over the ranks.  This module holds that host-side logic, written against
`torch.distributed` so that it runs over NCCL on GPUs and over gloo on CPU (which is how
it is tested):

* `shard` cuts the batch axis of an input, state, mask or upstream-gradient tensor;
* `dropconnect_mask` draws the recurrent-weight mask from a shared seed, because every rank
  must apply the same mask to its replica of the weights;
* `broadcast_parameters` makes the replicas identical at start;
* `all_reduce_tensors` / `all_reduce_gradients` sum gradients in flat buckets (one
  launch-latency-sized collective per bucket instead of one per tensor);
* `GradientBucket` is the flat buffer itself, handed to a backward op as its gradient
  outputs: the weight-gradient contractions and the bias column sums write straight into the
  buffer that the collective then reduces, with no pack before it and no scatter after;
* `attach` wires a whole network (`haste_b200.Stack` or single layers) for this: one bucket
  per layer and direction, its all-reduce started the moment that layer's backward pass has
  queued its weight-gradient contractions, so that the collective runs under the backward
  pass of the layers below and only the last one is exposed.

The reference has no multi-GPU path; its layers are used under the framework's own data
parallel wrappers, which this mirrors.
"""
import torch
import torch.distributed as dist

__all__ = ["shard", "dropconnect_mask", "broadcast_parameters", "all_reduce_tensors",
           "all_reduce_gradients", "GradientBucket", "attach", "DataParallel"]


def _world(group=None):
    if not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def shard(t, rank, world, batch_dim=1):
    """This rank's slice of `t` along the batch axis (`[T,N,...]` tensors: batch_dim=1,
    `[N,H]` states: batch_dim=0).  The batch must divide evenly: a ragged split would give the
    ranks different step times and the slowest one sets the pace."""
    if t is None:
        return None
    n = t.shape[batch_dim]
    if n % world:
        raise ValueError(f"batch of {n} does not divide over {world} ranks")
    per = n // world
    return t.narrow(batch_dim, rank * per, per).contiguous()


def dropconnect_mask(shape, drop_prob, seed, device=None, dtype=torch.float32):
    """Bernoulli(1 - drop_prob) keep-mask for the recurrent kernel, drawn on the CPU from
    `seed` alone so that every rank gets the same mask whatever its device state."""
    g = torch.Generator().manual_seed(int(seed))
    keep = torch.bernoulli(torch.full(tuple(shape), 1.0 - float(drop_prob)), generator=g)
    return keep.to(device=device, dtype=dtype)


def broadcast_parameters(module, src=0, group=None):
    """Copies rank `src`'s parameters and buffers to every rank, in place."""
    _, world = _world(group)
    if world == 1:
        return
    with torch.no_grad():
        for t in list(module.parameters()) + list(module.buffers()):
            dist.broadcast(t.data, src=src, group=group)


def all_reduce_tensors(tensors, group=None, bucket_bytes=64 << 20, async_op=False):
    """Sums each tensor of `tensors` over the ranks, in place.

    Tensors are packed into flat buckets of up to `bucket_bytes` per dtype; each bucket is one
    all-reduce.  With `async_op` the call returns a `finish()` callable: the collectives are in
    flight when it returns, and `finish()` waits for them and scatters the sums back - issue it
    after queuing the next layer's backward pass to overlap the two."""
    _, world = _world(group)
    tensors = [t for t in tensors if t is not None]
    if world == 1 or not tensors:
        return (lambda: None) if async_op else None
    buckets, cur, cur_bytes = [], [], 0
    for t in tensors:
        nbytes = t.numel() * t.element_size()
        if cur and (cur[0].dtype != t.dtype or cur[0].device != t.device
                    or cur_bytes + nbytes > bucket_bytes):
            buckets.append(cur)
            cur, cur_bytes = [], 0
        cur.append(t)
        cur_bytes += nbytes
    buckets.append(cur)
    pending = []
    for b in buckets:
        flat = torch.cat([t.reshape(-1) for t in b])
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
        pending.append((b, flat, work))

    def finish():
        for b, flat, work in pending:
            work.wait()
            off = 0
            for t in b:
                n = t.numel()
                t.copy_(flat[off:off + n].view_as(t))
                off += n

    if async_op:
        return finish
    finish()
    return None


def all_reduce_gradients(module_or_params, group=None, bucket_bytes=64 << 20, async_op=False):
    """Sums the `.grad` of every parameter over the ranks (see `all_reduce_tensors`)."""
    params = (module_or_params.parameters() if hasattr(module_or_params, "parameters")
              else module_or_params)
    return all_reduce_tensors([p.grad for p in params if p.grad is not None], group=group,
                              bucket_bytes=bucket_bytes, async_op=async_op)


_CELL_GATES = {"lstm": 4, "gru": 3, "indrnn": 1, "layer_norm_lstm": 4, "layer_norm_gru": 3,
               "layer_norm_indrnn": 1}


class GradientBucket:
    """One flat buffer that holds every parameter gradient of a layer (one direction).

    Pass it to a backward op (`ops.lstm_backward(..., grads=bucket)` and the like): the op
    takes its zero-initialised `dW`, `dR`, bias and LayerNorm-gain outputs as views of the
    buffer instead of allocating them, so the library's contractions write into the bucket
    directly, and `all_reduce` is then a single collective over memory that is already
    packed.  `reset` zeroes the buffer (the ops accumulate into their outputs) and rewinds it
    for the next step.  Views start on 256-byte boundaries, which the contraction's 16-byte
    stores need.
    """

    ALIGN_BYTES = 256

    def __init__(self, shapes, dtype, device):
        self.dtype = dtype
        self._align = self.ALIGN_BYTES // torch.empty((), dtype=dtype).element_size()
        total = sum(self._padded(_numel(s)) for s in shapes)
        self.flat = torch.zeros(max(total, 1), dtype=dtype, device=device)
        self._cursor = 0

    @classmethod
    def for_cell(cls, cell, input_size, hidden_size, dtype, device):
        """A bucket sized for the parameter gradients of one `cell` layer."""
        C, H, G = input_size, hidden_size, _CELL_GATES[cell]
        if "indrnn" in cell:
            shapes = [(C, H), (H,), (H,)]
        elif "gru" in cell:
            shapes = [(C, G * H), (H, G * H), (G * H,), (G * H,)]
        else:
            shapes = [(C, G * H), (H, G * H), (G * H,)]
        if cell.startswith("layer_norm"):
            shapes.append((2, G * H))
        if cell == "layer_norm_lstm":
            shapes += [(H,), (H,)]
        return cls(shapes, dtype, device)

    def _padded(self, n):
        return (n + self._align - 1) // self._align * self._align

    def reset(self):
        self.flat.zero_()
        self._cursor = 0

    def take(self, *shape):
        """The next `shape`-sized view of the buffer (zero after `reset`)."""
        if len(shape) == 1 and not isinstance(shape[0], int):
            shape = tuple(shape[0])
        n = _numel(shape)
        if self._cursor + n > self.flat.numel():
            raise ValueError("gradient bucket is too small for the outputs taken from it")
        view = self.flat[self._cursor:self._cursor + n].view(*shape)
        self._cursor += self._padded(n)
        return view

    def all_reduce(self, group=None, async_op=False):
        """Sums the buffer over the ranks, in place.  With `async_op` returns the work handle
        (or None on a single rank); wait on it before reading the views."""
        _, world = _world(group)
        if world == 1:
            return None
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
        if async_op:
            return work
        work.wait()
        return None


def _numel(shape):
    n = 1
    for d in shape:
        n *= int(d)
    return n


_CELL_OF_CLASS = {"LSTM": "lstm", "GRU": "gru", "IndRNN": "indrnn",
                  "LayerNormLSTM": "layer_norm_lstm", "LayerNormGRU": "layer_norm_gru",
                  "LayerNormIndRNN": "layer_norm_indrnn"}


class _LayerHook:
    """What a layer's autograd function sees of the data-parallel wiring: the bucket its
    backward op writes into, and `gradients_ready`, called once that op has been queued."""

    def __init__(self, owner, layer):
        cell = _CELL_OF_CLASS[type(layer).__name__]
        p = next(layer.parameters())
        self.owner, self.layer = owner, layer
        self.bucket = GradientBucket.for_cell(cell, layer.input_size, layer.hidden_size, p.dtype,
                                              p.device)
        self.recurrent_scale = None  # DropConnect mask / (1 - p) of the current step, if any
        self.views = None            # parameter name -> view of the bucket
        self.work = None

    def gradients_ready(self, views):
        self.views = views
        self.owner.order.append(self)
        if self.owner.overlap and self.owner.reduce:
            self.work = self.bucket.all_reduce(self.owner.group, async_op=True)


class DataParallel:
    """Batch-sharded data parallelism for a network of haste_b200 layers.

        dp = data_parallel.attach(net)          # after net.cuda(), inside an initialised group
        for step in ...:
            dp.zero_grad()
            y = net(shard(x, rank, world)); loss(y).backward()
            dp.finish()                         # gradients summed over the ranks, in p.grad
            optimiser.step()

    Every rank runs its slice of the batch; the parameter gradients of each layer and
    direction are written by that layer's backward pass straight into one flat buffer, whose
    all-reduce (NCCL: on the communicator's own stream) is issued as soon as the pass is queued
    and therefore overlaps the backward passes of the layers below it.  `finish` makes the
    current stream wait for the collectives and points every parameter's `.grad` at its summed
    view.  With DropConnect the buffer holds the gradient of the masked recurrent kernel; the
    mask (identical on every rank, see `dropconnect_mask`) is applied after the sum, which is
    the same by linearity.  `overlap=False` issues the collectives in `finish` instead (to
    measure what the overlap hides); `reduce=False` skips them.
    """

    def __init__(self, net, group=None, overlap=True, reduce=True):
        self.group, self.overlap, self.reduce = group, overlap, reduce
        self.hooks, self.order = [], []
        for m in net.modules():
            if type(m).__name__ in _CELL_OF_CLASS and hasattr(m, "_dp"):
                hook = _LayerHook(self, m)
                m._dp = hook
                self.hooks.append(hook)
        if not self.hooks:
            raise ValueError("no haste_b200 layer found in the module")

    def zero_grad(self):
        """Zeroes the buckets (the backward ops accumulate into them) and drops the layers'
        `.grad` references to them.  Call before each forward pass."""
        self.order = []
        for h in self.hooks:
            h.bucket.reset()
            h.views, h.work = None, None
            for p in h.layer.parameters():
                p.grad = None

    def bucket_bytes(self):
        return sum(h.bucket.flat.numel() * h.bucket.flat.element_size() for h in self.hooks)

    def finish(self):
        """Waits (on the current stream) for the gradient sums and installs them as `.grad`."""
        for h in self.order:
            if self.reduce and not self.overlap:
                h.work = h.bucket.all_reduce(self.group, async_op=True)
            if h.work is not None:
                h.work.wait()
                h.work = None
            for name, view in h.views.items():
                if name == "recurrent_kernel" and h.recurrent_scale is not None:
                    view = view * h.recurrent_scale
                getattr(h.layer, name).grad = view
        self.order = []

    def detach(self):
        for h in self.hooks:
            h.layer._dp = None


def attach(net, group=None, overlap=True, reduce=True):
    """Wires `net` (any module containing haste_b200 layers) for batch-sharded data
    parallelism; see `DataParallel`."""
    return DataParallel(net, group=group, overlap=overlap, reduce=reduce)
