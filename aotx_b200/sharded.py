"""The two places where the Q8_0 path shards over the GPUs of one box.

The reference is single-GPU, so nothing here mirrors reference code; the single-GPU results
are the contract.  One process per GPU, `torch.distributed` (NCCL over NVLink on GPUs, gloo in
the CPU tests) for the exchange steps.

* `ColumnSplit`: a large projection `y = x . w^T` split by rows of w (= columns of y).  Rows
  are independent and contiguous in the block layout, so a rank's shard is a plain byte range
  of the tensor; x is replicated; one all-gather of the y slices ends the step.
* `ExpertParallel`: routed experts with whole experts placed on ranks.  Tokens are sharded,
  routing is local, (token, rank) pairs travel to the expert's owner in one all-to-all, the
  owner runs the grouped expert products, the float results travel back in a second
  all-to-all, and the home rank forms the rank-ordered weighted sum exactly as on one GPU.

The compute step is injected (`product` / `experts`) so that the exchange logic runs on CPU
ranks in the tests; on GPUs it is the library's own kernels.
"""


def shard_rows(n, world, rank):
    """Rows [first, last) of an n-row tensor owned by `rank`: as even as possible, the first
    n % world ranks hold one row more."""
    base, extra = divmod(n, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def expert_owner(expert, experts, world):
    """The rank that holds `expert` under the same even split."""
    base, extra = divmod(experts, world)
    edge = extra * (base + 1)
    if expert < edge:
        return expert // (base + 1)
    return extra + (expert - edge) // base


def _dist():
    import torch.distributed as dist
    return dist


class ColumnSplit:
    """y[m][n] = x[m][k] . w[n][k]^T with the rows of w split over the ranks.

    `product(x, m) -> y_local[m][rows]` computes this rank's slice (on GPUs:
    `Q8Context.matmul` on the rank's byte range of w)."""

    def __init__(self, n, k, world, rank, product, group=None):
        self.n, self.k, self.world, self.rank = n, k, world, rank
        self.first, self.last = shard_rows(n, world, rank)
        self.rows = self.last - self.first
        self.max_rows = shard_rows(n, world, 0)[1]
        self.product = product
        self.group = group

    @staticmethod
    def shard_bytes(n, k, world, rank):
        """Byte range of this rank's rows in the Q8_0 tensor."""
        first, last = shard_rows(n, world, rank)
        stride = (k // 32) * 34
        return first * stride, last * stride

    def matmul(self, x, m, out=None):
        """Returns y[m][n], the same on every rank."""
        import torch
        y_local = self.product(x, m)
        if self.world == 1:
            return y_local
        even = self.n % self.world == 0
        if even:
            padded = y_local.contiguous()
        else:
            padded = y_local.new_zeros((m, self.max_rows))
            padded[:, :self.rows] = y_local
        gathered = y_local.new_empty((self.world, m, self.max_rows))
        _dist().all_gather(list(gathered.unbind(0)), padded, group=self.group)
        if out is None:
            out = y_local.new_empty((m, self.n))
        for r in range(self.world):
            first, last = shard_rows(self.n, self.world, r)
            out[:, first:last] = gathered[r, :, :last - first]
        return out


class ExpertParallel:
    """Routed feed-forward step with experts placed on ranks.

    `experts(x_pairs, local_expert_of_pair) -> proj[pairs][hidden]` (float) runs the expert
    products of this rank for the pairs it received (on GPUs: `Q8Context.moe_ffn` with one
    selection per row and weight 1).  `combine(proj[tokens][used][hidden], prob, ids) -> out`
    is the rank-ordered weighted sum (`Q8Context.moe_combine`)."""

    def __init__(self, experts_total, used, hidden, world, rank, experts, combine, group=None):
        self.experts_total, self.used, self.hidden = experts_total, used, hidden
        self.world, self.rank = world, rank
        self.first, self.last = shard_rows(experts_total, world, rank)
        self.experts = experts
        self.combine = combine
        self.group = group

    def ffn(self, x, prob, ids):
        """x: [tokens_local][hidden] half, prob: [tokens_local][experts_total] float,
        ids: [tokens_local][used] int32.  Returns out[tokens_local][hidden]."""
        import torch
        dist = _dist()
        tokens = x.shape[0]
        pairs = tokens * self.used
        flat = ids.reshape(-1).long()
        owner = torch.empty_like(flat)
        base, extra = divmod(self.experts_total, self.world)
        edge = extra * (base + 1)
        low = flat < edge
        owner[low] = flat[low] // (base + 1)
        if base > 0:
            owner[~low] = extra + (flat[~low] - edge) // base
        # pairs grouped by destination rank, stable, so that the way back is the inverse
        order = torch.argsort(owner, stable=True)
        send_counts = torch.bincount(owner, minlength=self.world)
        recv_counts = torch.empty_like(send_counts)
        if self.world > 1:
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        else:
            recv_counts.copy_(send_counts)
        send_list = send_counts.tolist()
        recv_list = recv_counts.tolist()
        rows_out = x[(order // self.used)]
        expert_out = flat[order].to(torch.int32)
        got = int(sum(recv_list))
        rows_in = x.new_empty((got, self.hidden))
        expert_in = expert_out.new_empty((got,))
        if self.world > 1:
            dist.all_to_all_single(rows_in, rows_out.contiguous(), recv_list, send_list, group=self.group)
            dist.all_to_all_single(expert_in, expert_out.contiguous(), recv_list, send_list, group=self.group)
        else:
            rows_in.copy_(rows_out)
            expert_in.copy_(expert_out)
        proj_in = self.experts(rows_in, expert_in - self.first)
        proj_back = proj_in.new_empty((pairs, self.hidden))
        if self.world > 1:
            dist.all_to_all_single(proj_back, proj_in.contiguous(), send_list, recv_list, group=self.group)
        else:
            proj_back.copy_(proj_in)
        proj = proj_back.new_empty((pairs, self.hidden))
        proj[order] = proj_back
        return self.combine(proj.reshape(tokens, self.used, self.hidden), prob, ids)


def column_split_on_gpu(ctx, w_local, n, k, world, rank, y_dtype=None, group=None):
    """`ColumnSplit` whose local step is the library's product on this rank's rows of w
    (`w_local`: device tensor holding the byte range `ColumnSplit.shard_bytes`)."""
    first, last = shard_rows(n, world, rank)

    def product(x, m):
        return ctx.matmul(w_local, last - first, k, x, m=m, y_dtype=y_dtype)

    return ColumnSplit(n, k, world, rank, product, group=group)


def expert_parallel_on_gpu(ctx, w_gate, w_up, w_down, experts_total, used, hidden, ffn, world, rank,
                           group=None):
    """`ExpertParallel` whose local step is the library's grouped expert products on this
    rank's experts (`w_*`: device tensors holding only those experts' slices)."""
    import torch
    first, last = shard_rows(experts_total, world, rank)
    local = last - first

    def experts(rows, local_expert):
        count = rows.shape[0]
        if count == 0:
            return torch.zeros((0, hidden), dtype=torch.float32, device=rows.device)
        ones = torch.ones((count, local), dtype=torch.float32, device=rows.device)
        ids = local_expert.to(torch.int32).reshape(count, 1).contiguous()
        return ctx.moe_ffn(w_gate, w_up, w_down, local, hidden, ffn, rows.contiguous(), ones, ids,
                           tokens=count)

    def combine(proj, prob, ids):
        return ctx.moe_combine(proj.contiguous(), prob, ids)

    return ExpertParallel(experts_total, used, hidden, world, rank, experts, combine, group=group)


class ColumnSplitFused:
    """Column-split projection whose gather happens in the product's own stores.

    y lives in symmetric memory (`torch.distributed._symmetric_memory`): every rank can store
    into every rank's copy.  The kernel of rank r writes its column slice of each tile into all
    copies (plain stores over NVLink, no multicast loads), and one device-side barrier orders
    the ranks before anyone reads y.

    There are two copies of y, used by alternate steps, and that is what makes one barrier per
    step enough: a rank that writes the buffer of step s + 2 has passed the barrier of step
    s + 1, which every rank reaches only after its own product of step s + 1, and that product
    follows, on the rank's stream, whatever the rank read from the buffer of step s.  So no
    store can land in a buffer that a peer still reads.  The result of a step is a view that
    stays valid until the step after the next one.

    A call that is captured into a CUDA graph uses, on every replay, the buffer it was captured
    with, so the argument above does not cover it: such a call is opened by a barrier as well
    (`opening_barrier=None` decides by whether the stream is capturing).  A caller whose graph
    holds another barrier of the same ranks between two uses of one buffer - as a rotation over
    two or more of these objects does - may pass `opening_barrier=False`: a rank leaves that
    barrier only after every peer has reached it, and a peer reaches it only after what it read
    from the buffer before."""

    def __init__(self, ctx, w_local, n, k, world, rank, m_max, y_dtype, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.ctx, self.w_local = ctx, w_local
        self.n, self.k, self.world, self.rank = n, k, world, rank
        self.first, self.last = shard_rows(n, world, rank)
        self.y_dtype = y_dtype
        group = group if group is not None else dist.group.WORLD
        self.y = symm.empty((2, m_max, n), dtype=y_dtype, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm.rendezvous(self.y, group)
        half = m_max * n * self.y.element_size()
        self.ptrs = [[int(p) + which * half for p in self.handle.buffer_ptrs] for which in (0, 1)]
        self.step = 0
        # nobody stores into a peer before every rank has its buffers
        self.handle.barrier(channel=0)

    def matmul(self, x, m, opening_barrier=None):
        import torch
        which = self.step & 1
        self.step += 1
        if opening_barrier is None:
            opening_barrier = torch.cuda.is_current_stream_capturing()
        if opening_barrier:
            self.handle.barrier(channel=which ^ 1)
        self.ctx.matmul_peers(self.w_local, self.last - self.first, self.k, x, m, self.ptrs[which], self.n,
                              self.first, self.y_dtype)
        self.handle.barrier(channel=which)
        return self.y[which, :m]
