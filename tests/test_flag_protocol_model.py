"""The cross-rank flag protocol of the fused FSDP2 path, model-checked on the host.

The host-side objects that assign epochs and channels (``_Pool``, ``PeerGradients``,
``ParamPush``) are the real ones; the device is replaced by a small simulator in which every
rank executes its queue of device operations in order and ranks interleave at random between
the phases of a kernel (publish ready / wait for all / read the ranks' buffers / store the
new parameters to every rank / publish done and pushed).  Whatever the interleaving:

* a kernel reads, from every rank, the gradients of its own step and group;
* a rank never overwrites a buffer that a peer's kernel is still reading;
* an all-gather served by the pushes sees every rank's parameters of the latest update;
* nothing deadlocks.

No GPU is involved; this is the stand-in for a race detector on the protocol level.
"""

import random
from types import SimpleNamespace

import pytest

from flashoptim_b200.parallel.fsdp import _Pool
from flashoptim_b200.parallel.symm import ParamPush

MAX_PEERS = 8


class _Args:
    def __init__(self, world, rank, buf, epoch, ready, done):
        self.world, self.rank, self.buf, self.epoch = world, rank, buf, epoch
        self.ready_channel, self.done_channel = ready, done
        self.multicast = None
        self.push = 0
        self.param_out = [None] * MAX_PEERS
        self.param_out_mc = None
        self.param_out_delta = 0
        self.push_epoch = 0
        self.pushed_channel = -1


class _SimGroup:
    """What ``PeerGroup`` is to the host code: hands out buffers and channels, records the
    device operations a rank enqueues."""

    def __init__(self, world, rank):
        self.world, self.rank = world, rank
        self.ops = []
        self._buffers = 0
        self._channels = 0

    def allocate(self, nbytes, zero=False):
        self._buffers += 1
        # "pointers" are (owner rank, buffer number): the same buffer number on every rank
        return SimpleNamespace(id=self._buffers, ptrs=[(r, self._buffers) for r in range(self.world)],
                               multicast_ptr=0)

    def new_channel(self):
        self._channels += 1
        return self._channels - 1

    def new_channels(self):
        self._channels += 2
        return self._channels - 2, self._channels - 1

    def comm_args(self, buf, epoch, ready, done, grad_out=None, grad_out_sub=0):
        return _Args(self.world, self.rank, buf, epoch, ready, done)

    def wait(self, args, channel):
        self.ops.append(("wait", channel, args.epoch))


class _Device:
    """Shared state of the simulated node."""

    def __init__(self, world):
        self.world = world
        self.flags = [dict() for _ in range(world)]      # per destination rank: (channel, src) -> epoch
        self.buffers = {}                                # (owner, buffer id) -> content tag
        self.pushed = {}                                 # (owner, buffer id, src rank) -> step
        self.reading = {}                                # reader rank -> set of (owner, buffer id)

    def flag(self, dst, channel, src):
        return self.flags[dst].get((channel, src), 0)


def _rank_program(dev, group, queue, errors):
    """Generator: executes the rank's device queue in order, yielding between atomic phases
    (``None`` = made progress, ``"blocked"`` = waiting for a flag)."""
    r, w = group.rank, group.world
    for op in queue:
        kind = op[0]
        if kind == "wait":
            _, channel, epoch = op
            while any(dev.flag(r, channel, s) < epoch for s in range(w)):
                yield "blocked"
        elif kind == "write":
            _, buf, tag = op
            for reader, held in dev.reading.items():
                if (r, buf.id) in held:
                    errors.append(f"rank {r} overwrites buffer {buf.id} while rank {reader} reads it")
            dev.buffers[(r, buf.id)] = tag
        elif kind == "kernel":
            _, a, tag, step = op
            for d in range(w):
                dev.flags[d][(a.ready_channel, r)] = a.epoch
            yield None
            while any(dev.flag(r, a.ready_channel, s) < a.epoch for s in range(w)):
                yield "blocked"
            dev.reading[r] = {(s, a.buf.id) for s in range(w)}
            for s in range(w):
                yield None
                got = dev.buffers.get((s, a.buf.id))
                if got != tag:
                    errors.append(f"rank {r} read {got} from rank {s}, expected {tag}")
            if a.push:
                for d in range(w):
                    yield None
                    owner, buf_id = a.param_out[d]
                    dev.pushed[(owner, buf_id, r)] = step
            dev.reading[r] = set()
            yield None
            for d in range(w):
                dev.flags[d][(a.done_channel, r)] = a.epoch
                if a.push:
                    dev.flags[d][(a.pushed_channel, r)] = a.push_epoch
        elif kind == "gather":
            _, buf, step = op
            for s in range(w):
                yield None
                got = dev.pushed.get((r, buf.id, s))
                if got != step:
                    errors.append(f"rank {r}: all-gather sees step {got} of rank {s}'s parameters, expected {step}")
        yield None


def _host_queue(group, n_groups, depth, steps, push):
    """What one rank's host code enqueues: the real pool / epoch objects drive it."""
    pool = _Pool(group, 1024, depth)
    targets = [ParamPush(group.allocate(1024), group.new_channel()) for _ in range(n_groups)] if push else []
    for step in range(1, steps + 1):
        if push and step > 1:
            for k in range(n_groups):                # forward all-gathers of this step
                t = targets[k]
                group.wait(group.comm_args(t.buf, t.epoch, t.channel, t.channel), t.channel)
                group.ops.append(("gather", t.buf, step - 1))
        for k in reversed(range(n_groups)):          # backward: one reduce-scatter per group
            if push and step > 1:                    # backward all-gather (resharded after forward)
                t = targets[k]
                group.wait(group.comm_args(t.buf, t.epoch, t.channel, t.channel), t.channel)
                group.ops.append(("gather", t.buf, step - 1))
            slot = pool.take()
            slot.wait_done()
            group.ops.append(("write", slot.buf, (step, k)))
            slot.push = targets[k] if push else None
            group.ops.append(("kernel", slot.next_args(), (step, k), step))
            slot.push = None
    return group.ops


@pytest.mark.parametrize("world", [2, 3, 4])
@pytest.mark.parametrize("n_groups,depth", [(1, 1), (2, 1), (3, 2), (4, 2), (3, 3)])
@pytest.mark.parametrize("push", [False, True])
def test_no_interleaving_breaks_the_protocol(world, n_groups, depth, push):
    for seed in range(25):
        rng = random.Random(1000 * seed + 17 * world + n_groups)
        dev = _Device(world)
        errors = []
        groups = [_SimGroup(world, r) for r in range(world)]
        programs = [_rank_program(dev, g, _host_queue(g, n_groups, depth, 3, push), errors) for g in groups]
        alive = set(range(world))
        blocked_in_a_row = 0
        while alive:
            r = rng.choice(sorted(alive))
            # bursts: a rank often runs far ahead of the others
            for _ in range(rng.choice([1, 1, 2, 5, 40])):
                try:
                    state = next(programs[r])
                except StopIteration:
                    alive.discard(r)
                    break
                if state == "blocked":
                    blocked_in_a_row += 1
                    break
                blocked_in_a_row = 0
            assert blocked_in_a_row < 200 * world, f"deadlock (seed {seed}): ranks {sorted(alive)} all wait"
        assert not errors, (seed, errors[:3])


def test_the_model_notices_a_missing_wait():
    """Sanity of the checker itself: without ``wait_done`` before a buffer is reused, some
    interleaving overwrites gradients that a slower peer has not read yet."""
    world, found = 2, False
    for seed in range(200):
        rng = random.Random(seed)
        dev = _Device(world)
        errors = []
        groups = [_SimGroup(world, r) for r in range(world)]
        queues = []
        for g in groups:
            q = [op for op in _host_queue(g, 2, 1, 3, False) if op[0] != "wait"]
            queues.append(q)
        programs = [_rank_program(dev, g, q, errors) for g, q in zip(groups, queues)]
        alive, spins = set(range(world)), 0
        while alive and spins < 10000:
            r = rng.choice(sorted(alive))
            for _ in range(rng.choice([1, 5, 40])):
                try:
                    if next(programs[r]) == "blocked":
                        spins += 1
                        break
                except StopIteration:
                    alive.discard(r)
                    break
        if errors:
            found = True
            break
    assert found


# ---------------------------------------------------------------------------------------------
# Fused DDP: buckets of one backward pass share one arena, and DDP rebuilds its buckets after
# the first iteration, so the regions of consecutive passes overlap at different offsets.


def _ddp_stream_program(dev, rank, world, queue, errors):
    """One CUDA stream of one rank.  The hook copies buckets into the arena on the stream that
    autograd runs on ("write" ops, preceded by the waits the layout asked for); the kernels run
    on a side stream and each starts only after its own bucket was written (an event).
    ``dev.buffers[owner]`` maps (offset, length) -> tag; ``dev.reading[reader]`` holds the
    (owner, offset, length) a running kernel still reads."""
    for op in queue:
        kind = op[0]
        if kind == "wait":
            _, epoch = op
            while any(dev.flag(rank, "done", s) < epoch for s in range(world)):
                yield "blocked"
        elif kind == "write":
            _, off, n, tag, epoch = op
            for reader, held in dev.reading.items():
                for owner, o, m in held:
                    if owner == rank and o < off + n and off < o + m:
                        errors.append(f"rank {rank} overwrites [{off},{off + n}) while rank {reader} reads [{o},{o + m})")
            mine = dev.buffers.setdefault(rank, {})
            for (o, m) in [k for k in mine if k[0] < off + n and off < k[0] + k[1]]:
                del mine[(o, m)]
            mine[(off, n)] = tag
            dev.pushed[("written", rank)] = epoch  # the event the side stream waits for
        elif kind == "kernel":
            _, epoch, off, n, tag = op
            while dev.pushed.get(("written", rank), 0) < epoch:
                yield "blocked"
            for d in range(world):
                dev.flags[d][("ready", rank)] = epoch
            yield None
            while any(dev.flag(rank, "ready", s) < epoch for s in range(world)):
                yield "blocked"
            dev.reading[("k", rank)] = {(s, off, n) for s in range(world)}
            for s in range(world):
                yield None
                got = dev.buffers.get(s, {}).get((off, n))
                if got != tag:
                    errors.append(f"rank {rank} read {got} from rank {s} at {off}, expected {tag}")
            dev.reading[("k", rank)] = set()
            yield None
            for d in range(world):
                dev.flags[d][("done", rank)] = epoch
        yield None


def _ddp_host_queues(layouts, place):
    """``layouts[step]`` = bucket sizes of that backward pass; ``place(index, nbytes, last_epoch)``
    is the arena bookkeeping under test.  Returns the (autograd stream, side stream) queues."""
    main, side, epoch = [], [], 0
    for step, sizes in enumerate(layouts):
        for index, n in enumerate(sizes):
            off, wait_epoch = place(index, n, epoch)
            if wait_epoch:
                main.append(("wait", wait_epoch))
            epoch += 1
            main.append(("write", off, n, (step, index), epoch))
            side.append(("kernel", epoch, off, n, (step, index)))
    return main, side


def _run_ddp_model(world, layouts, make_place, seeds):
    for seed in seeds:
        rng = random.Random(seed)
        dev = _Device(world)
        errors = []
        programs = []
        for r in range(world):
            main, side = _ddp_host_queues(layouts, make_place())
            programs.append(_ddp_stream_program(dev, r, world, main, errors))
            programs.append(_ddp_stream_program(dev, r, world, side, errors))
        alive, blocked = set(range(len(programs))), 0
        while alive:
            i = rng.choice(sorted(alive))
            for _ in range(rng.choice([1, 1, 2, 5, 40])):
                try:
                    state = next(programs[i])
                except StopIteration:
                    alive.discard(i)
                    break
                if state == "blocked":
                    blocked += 1
                    break
                blocked = 0
            assert blocked < 400 * world, f"deadlock (seed {seed})"
        if errors:
            return errors
    return []


# First pass: buckets in the order of registration; afterwards DDP's rebuilt buckets (other
# sizes, hence other offsets for everything but the first).
_DDP_LAYOUTS = [[512, 1024, 256], [768, 1024], [512, 512, 1024], [256, 1536], [256, 1536]]


@pytest.mark.parametrize("world", [2, 3, 4])
def test_ddp_arena_survives_rebuilt_buckets(world):
    from flashoptim_b200.parallel.ddp import ArenaLayout

    errors = _run_ddp_model(world, _DDP_LAYOUTS, lambda: ArenaLayout(4096).place, range(40))
    assert not errors, errors[:3]


def test_the_ddp_model_notices_protection_keyed_by_offset():
    """Control: waiting only for the last use of the SAME offset (what an exact-offset map does)
    lets a rebuilt bucket overwrite a region that a slower peer still reads."""

    def make_place():
        cursor, last_use = [0], {}

        def place(index, nbytes, last_epoch):
            if index == 0:
                cursor[0] = 0
            off = cursor[0]
            cursor[0] += (nbytes + 255) // 256 * 256
            wait_epoch = last_use.get(off, 0)
            last_use[off] = last_epoch + 1  # the epoch this bucket's kernel will get
            return off, wait_epoch

        return place

    assert _run_ddp_model(2, _DDP_LAYOUTS, make_place, range(200))
