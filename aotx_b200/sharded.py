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

    `experts(x_rows, local_expert_of_row) -> proj[rows][hidden]` (float) runs the expert products
    of this rank for the rows it received; a row whose expert number lies outside
    [0, local experts) is padding and its result is never read (on GPUs: `Q8Context.moe_ffn` with
    one selection per row and weight 1, which leaves such rows out).  `combine(proj[tokens][used]
    [hidden], prob, ids) -> out` is the rank-ordered weighted sum (`Q8Context.moe_combine`).

    Every buffer of the exchange has a fixed size (room for all of a rank's pairs towards every
    destination), the counts never come to the host, and the padding carries an expert number
    that names no expert, so the whole step is a fixed sequence of device operations and can be
    captured in a CUDA graph.  A selection outside the expert table (ids >= experts_total) is
    dropped on every rank alike and adds nothing to its token's sum, as on one GPU."""

    PADDING = 0x7FFFFFF0  # an expert number no rank holds

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
        world = self.world
        tokens = x.shape[0]
        pairs = tokens * self.used
        flat = ids.reshape(-1).long()
        valid = (flat >= 0) & (flat < self.experts_total)
        base, extra = divmod(self.experts_total, world)
        edge = extra * (base + 1)
        owner_low = flat // (base + 1)
        owner_high = extra + (flat - edge) // max(base, 1)
        owner = torch.where(flat < edge, owner_low, owner_high)
        owner = torch.where(valid, owner, torch.full_like(owner, world))      # bucket `world`: dropped
        # pairs grouped by destination rank, stable, so that the way back is the inverse
        order = torch.argsort(owner, stable=True)
        owner_sorted = owner[order]
        counts = torch.zeros(world + 1, dtype=torch.long, device=x.device)
        counts.scatter_add_(0, owner, torch.ones_like(owner))
        starts = torch.cumsum(counts, 0) - counts
        place = torch.arange(pairs, device=x.device) - starts[owner_sorted]    # position within its destination
        keep = owner_sorted < world
        slot = torch.where(keep, owner_sorted * pairs + place, torch.full_like(place, world * pairs))
        # one segment of `pairs` rows per destination (and one spare row that takes what is dropped)
        rows_out = x.new_zeros((world * pairs + 1, self.hidden))
        expert_out = torch.full((world * pairs + 1,), self.PADDING, dtype=torch.int32, device=x.device)
        rows_out[slot] = x[order // self.used]
        expert_out[slot] = torch.where(keep, flat[order], torch.full_like(flat, self.PADDING)).to(torch.int32)
        rows_out, expert_out = rows_out[:world * pairs], expert_out[:world * pairs]
        if world > 1:
            rows_in = torch.empty_like(rows_out)
            expert_in = torch.empty_like(expert_out)
            dist.all_to_all_single(rows_in, rows_out, group=self.group)
            dist.all_to_all_single(expert_in, expert_out, group=self.group)
        else:
            rows_in, expert_in = rows_out, expert_out
        proj_in = self.experts(rows_in, expert_in - self.first)
        if world > 1:
            proj_back = torch.empty_like(proj_in)
            dist.all_to_all_single(proj_back, proj_in.contiguous(), group=self.group)
        else:
            proj_back = proj_in
        # the result of a pair that was dropped is zero; the others come back from their slot
        spare = torch.cat([proj_back, proj_back.new_zeros((1, self.hidden))])
        proj = proj_back.new_zeros((pairs, self.hidden))
        proj[order] = spare[slot]
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

    state = {}

    def experts(rows, local_expert):
        # every row carries one selection with weight 1; padding rows name no local expert and
        # are left out of the products (their result rows are never read)
        count = rows.shape[0]
        if "ones" not in state or state["ones"].shape[0] != count:
            state["ones"] = torch.ones((count, local), dtype=torch.float32, device=rows.device)
            state["workspace"] = ctx.moe_workspace(count, 1, hidden, ffn)
            state["out"] = torch.zeros((count, hidden), dtype=torch.float32, device=rows.device)
        ids = local_expert.to(torch.int32).reshape(count, 1).contiguous()
        return ctx.moe_ffn(w_gate, w_up, w_down, local, hidden, ffn, rows.contiguous(), state["ones"], ids,
                           tokens=count, out=state["out"], workspace=state["workspace"])

    def combine(proj, prob, ids):
        return ctx.moe_combine(proj.contiguous(), prob, ids)

    return ExpertParallel(experts_total, used, hidden, world, rank, experts, combine, group=group)


class ColumnSplitFused:
    """Column-split projection whose gather happens in the product's own stores
    (`aotx_q8_matmul_colsplit`).

    y and a small array of flag words live in symmetric memory
    (`torch.distributed._symmetric_memory`, used only to allocate and exchange the addresses):
    every rank can store into every rank's copy.  The kernel of rank r writes its column slice of
    each tile into all copies (plain stores over NVLink, no multicast loads), and the library's
    own barrier - each rank writes a step number into its word of every rank's flag array and
    waits, with a bound, until its own array has reached it - orders the ranks before anyone
    reads y.  No library kernel sits on the step's path.

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
        device = torch.device("cuda", torch.cuda.current_device())
        self.y = symm.empty((2, m_max, n), dtype=y_dtype, device=device)
        self.handle = symm.rendezvous(self.y, group)
        half = m_max * n * self.y.element_size()
        self.ptrs = [[int(p) + which * half for p in self.handle.buffer_ptrs] for which in (0, 1)]
        # one flag word per source rank, and this rank's step counter
        self.flags = symm.empty((max(world, 8),), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flag_handle = symm.rendezvous(self.flags, group)
        self.flag_ptrs = [int(p) for p in self.flag_handle.buffer_ptrs]
        self.step_word = torch.zeros(1, dtype=torch.int32, device=device)
        self.step = 0
        torch.cuda.synchronize()
        # nobody stores into a peer before every rank has its buffers and zeroed flags (set-up only)
        self.handle.barrier(channel=0)

    def barrier(self):
        self.ctx.peer_barrier(self.flag_ptrs, self.rank, self.step_word)

    def matmul(self, x, m, opening_barrier=None):
        import torch
        which = self.step & 1
        self.step += 1
        if opening_barrier is None:
            opening_barrier = torch.cuda.is_current_stream_capturing()
        if opening_barrier:
            self.barrier()
        self.ctx.matmul_colsplit(self.w_local, self.last - self.first, self.k, x, m, self.ptrs[which],
                                 self.flag_ptrs, self.rank, self.n, self.first, self.y_dtype, self.step_word)
        return self.y[which, :m]


class ExpertParallelFused:
    """The routed step with experts placed on ranks and the exchange folded into the library's
    own kernels (`aotx_q8_moe_ep`): no all-to-all, no staging buffers, no library collective.

    Every rank keeps its tokens' activations and selections, and the projections of its experts,
    in symmetric memory (`torch.distributed._symmetric_memory`, used only to allocate and to
    exchange the addresses).  Per step and rank, one call: barrier, gather of the rows of the
    pairs that name a local expert straight from the GPU that holds the token, the grouped
    products, barrier, and the rank-ordered sum that reads every pair's projection from the GPU
    that computed it (plain loads over NVLink).  The first barrier of step s + 1 is also what
    keeps a fast rank from overwriting projections that a peer still sums: it is passed only
    when every rank has finished step s."""

    def __init__(self, ctx, w_gate, w_up, w_down, experts_total, used, hidden, ffn, world, rank, tokens,
                 group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.ctx = ctx
        self.w = (w_gate, w_up, w_down)
        self.experts_total, self.used, self.hidden, self.ffn_rows = experts_total, used, hidden, ffn
        self.world, self.rank, self.tokens = world, rank, tokens
        group = group if group is not None else dist.group.WORLD
        device = torch.device("cuda", torch.cuda.current_device())
        self.x = symm.empty((tokens, hidden), dtype=torch.float16, device=device)
        self.ids = symm.empty((tokens, used), dtype=torch.int32, device=device)
        self.proj = symm.empty((world * tokens * used, hidden), dtype=torch.float32, device=device)
        self.flags = symm.empty((max(world, 8),), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.proj.zero_()
        handles = [symm.rendezvous(t, group) for t in (self.x, self.ids, self.proj, self.flags)]
        self.x_ptrs, self.ids_ptrs, self.proj_ptrs, self.flag_ptrs = (
            [int(p) for p in h.buffer_ptrs] for h in handles)
        self.step_word = torch.zeros(1, dtype=torch.int32, device=device)
        self.workspace = ctx.moe_ep_workspace(tokens, used, hidden, ffn, world)
        self.out = torch.empty((tokens, hidden), dtype=torch.float32, device=device)
        torch.cuda.synchronize()
        # nobody signals a peer before every rank has its buffers and zeroed flags (set-up only)
        handles[0].barrier(channel=0)

    def ffn(self, x, prob, ids):
        """x: [tokens][hidden] half, prob: [tokens][experts_total] float, ids: [tokens][used]
        int32 - this rank's tokens.  Returns out[tokens][hidden] (valid until the next call)."""
        self.x.copy_(x)
        self.ids.copy_(ids)
        return self.ctx.moe_ep(*self.w, self.experts_total, self.hidden, self.ffn_rows, self.x_ptrs, self.ids_ptrs,
                               prob, self.tokens, self.used, self.proj_ptrs, self.flag_ptrs, self.rank,
                               self.step_word, self.out, self.workspace)
