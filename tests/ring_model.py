"""Random-interleaving model of the decode-regime kernel's ring protocol (test infrastructure).

The kernels hand stages of shared and tensor memory between warps through mbarriers that are
waited on by phase parity.  A parity wait cannot tell a phase from the one two phases later,
so a ring is only safe if no waiter can get two phases ahead of the barrier it polls.  These
model runs the barrier protocol of aotx_b200/csrc/q8_stream.cu (same counts,
same parity formulas, same order of waits and arrivals per warp) as cooperating generators
under a random scheduler, with copies and MMAs completing asynchronously after random delays,
and record any read of a stage that does not hold the expected piece."""
import random


class Barrier:
    """mbarrier: `count` arrivals plus outstanding copy bytes complete a phase."""

    def __init__(self, count):
        self.count = count
        self.pending = count
        self.tx = 0
        self.phase = 0

    def _advance(self):
        if self.pending == 0 and self.tx == 0:
            self.phase += 1
            self.pending = self.count

    def arrive(self):
        assert self.pending > 0, "more arrivals than the barrier was made for"
        self.pending -= 1
        self._advance()

    def expect(self, amount):
        self.tx += amount
        self.arrive()

    def complete(self, amount):
        self.tx -= amount
        self._advance()

    def passed(self, parity):
        """try_wait.parity: true once the phase of that parity has completed."""
        return (self.phase & 1) != parity


class Machine:
    def __init__(self, seed):
        self.rnd = random.Random(seed)
        self.clock = 0
        self.timers = []
        self.errors = []
        self.mma_queue = []

    def later(self, fn, low=1, high=40):
        self.timers.append((self.clock + self.rnd.randint(low, high), fn))

    def tensor_core(self):
        """Queued MMAs execute in order, each some time after it was issued."""
        while True:
            if self.mma_queue:
                for _ in range(self.rnd.randint(0, 6)):
                    yield
                self.mma_queue.pop(0)()
            yield

    def run(self, agents, limit=3_000_000):
        agents = list(agents) + [self.tensor_core()]
        alive = [True] * len(agents)
        steps = 0
        while any(alive[:-1]) or self.mma_queue:
            self.clock += 1
            steps += 1
            if steps > limit:
                self.errors.append(("no progress",))
                break
            due = [t for t in self.timers if t[0] <= self.clock]
            if due:
                self.timers = [t for t in self.timers if t[0] > self.clock]
                for _, fn in due:
                    fn()
            i = self.rnd.randrange(len(agents))
            if alive[i]:
                try:
                    next(agents[i])
                except StopIteration:
                    alive[i] = False
            if self.errors:
                break
        return self.errors


def weight_producer(mach, raw, raw_full, raw_empty, pieces):
    stages = len(raw)
    for g in range(pieces):
        st, ph = g % stages, (g // stages) & 1
        while not raw_empty[st].passed(ph ^ 1):
            yield
        raw_full[st].expect(1)
        raw[st] = ("in flight", g)

        def land(st=st, g=g):
            raw[st] = g
            raw_full[st].complete(1)

        mach.later(land)
        yield


def stream_kernel(seed, raw_stages, depth, segments, bf16):
    """q8_stream_kernel: A stages in tensor memory, one hand-over per 256-deep segment."""
    mach = Machine(seed)
    raw = [None] * raw_stages
    raw_full = [Barrier(1) for _ in range(raw_stages)]
    raw_empty = [Barrier(8) for _ in range(raw_stages)]
    xs = [None] * depth
    x_ready = [dict() for _ in range(depth)]   # bf16: which converter warps have converted
    x_full = [Barrier(1) for _ in range(depth)]
    a_slots = [dict() for _ in range(depth)]
    a_full = [Barrier(8) for _ in range(depth)]
    seg_empty = [Barrier(1) for _ in range(depth)]

    def x_producer():
        for g in range(segments):
            st, ph = g % depth, (g // depth) & 1
            while not seg_empty[st].passed(ph ^ 1):
                yield
            x_full[st].expect(1)
            xs[st] = ("in flight", g)

            def land(st=st, g=g):
                xs[st] = g
                x_full[st].complete(1)

            mach.later(land)
            yield

    def issuer():
        for g in range(segments):
            st, ph = g % depth, (g // depth) & 1
            while not a_full[st].passed(ph):
                yield
            while not x_full[st].passed(ph):
                yield

            def execute(st=st, g=g):
                for cw in range(8):
                    if a_slots[st].get(cw) != g:
                        mach.errors.append(("A stage", g, st, cw, a_slots[st].get(cw)))
                    if bf16 and x_ready[st].get(cw) != g:
                        mach.errors.append(("x not converted", g, st, cw, x_ready[st].get(cw)))
                if xs[st] != g:
                    mach.errors.append(("x stage", g, xs[st]))
                seg_empty[st].arrive()

            mach.mma_queue.append(execute)
            yield

    def converter(cw):
        for g in range(segments):
            rst, rph = g % raw_stages, (g // raw_stages) & 1
            while not raw_full[rst].passed(rph):
                yield
            for _ in range(mach.rnd.randint(0, 3)):
                yield
            if raw[rst] != g:
                mach.errors.append(("raw stage", g, raw[rst], cw))
            raw_empty[rst].arrive()
            st, ph = g % depth, (g // depth) & 1
            while not seg_empty[st].passed(ph ^ 1):
                yield
            for _ in range(mach.rnd.randint(0, 4)):
                yield
            a_slots[st][cw] = g
            if bf16:
                while not x_full[st].passed(ph):
                    yield
                if xs[st] != g:
                    mach.errors.append(("x read early", g, xs[st], cw))
                x_ready[st][cw] = g
            a_full[st].arrive()
            yield

    agents = [weight_producer(mach, raw, raw_full, raw_empty, segments), x_producer(), issuer()]
    agents += [converter(c) for c in range(8)]
    return mach.run(agents)
