"""CPU model of the mbarrier protocols of the tensor-core kernels.

Each role of a kernel (TMA producer, converter warps, MMA issuer, epilogue) is replayed as a
coroutine that performs the same sequence of barrier operations as the CUDA code, under a
random scheduler and with TMA loads that complete in ANY order.  The model checks what a GPU
run cannot show cheaply:

* no role can dead-lock;
* no barrier receives more arrivals in a phase than it was initialised for;
* every parity wait is unambiguous: at each poll, "the phase with this parity bit has
  completed" (what the hardware answers) must equal "the phase this waiter means has
  completed" (what the code relies on).  A parity bit cannot tell phase k from phase k-2, so a
  waiter that polls a barrier whose phase k-1 is still open gets a false "done".

mbarrier model: `count` arrivals per phase, a transaction-byte balance that may go negative
(bytes may land before the expect_tx of their phase), a count of completed phases.  On a fresh
barrier wait(parity 1) passes at once (the producers' first pass over the ring).

The last rule is why converter groups own pipeline STAGES (stage s belongs to group s % G) and
not rounds (round i to group i % G): with rounds dealt round-robin and a stage count that is no
multiple of G, a group meets a stage's barrier only every few phases, and an out-of-order TMA
completion lets it poll while the previous phase is open.  `test_round_robin_groups_are_ambiguous`
keeps that counter-example."""
import random

import pytest


class ProtocolError(AssertionError):
    pass


class Barrier:
    def __init__(self, name, count):
        self.name, self.count = name, count
        self.pending, self.tx, self.phases_done = count, 0, 0

    def _maybe_complete(self):
        if self.pending == 0 and self.tx == 0:
            self.phases_done += 1
            self.pending = self.count

    def arrive(self, tx=0):
        if self.pending <= 0:
            raise ProtocolError(f"{self.name}: more arrivals than the barrier was initialised for")
        self.tx += tx
        self.pending -= 1
        self._maybe_complete()

    def complete_tx(self, nbytes):
        self.tx -= nbytes
        self._maybe_complete()

    def poll(self, parity, need):
        """try_wait(parity) as the hardware answers it; `need` = number of completed phases the
        waiter actually relies on.  Raises when the two disagree."""
        hw = (parity == 1) if self.phases_done == 0 else (((self.phases_done - 1) & 1) == parity)
        meant = self.phases_done >= need
        if hw != meant or self.phases_done > need:
            raise ProtocolError(
                f"{self.name}: ambiguous parity wait (completed phases {self.phases_done}, waiter needs {need})")
        return hw


def consumer_wait(bar, use):   # k-th use of the barrier, waits for phase k: parity k & 1
    return (bar, use & 1, use + 1)


def producer_wait(bar, use):   # k-th refill, waits for release k-1: inverted parity, passes at once for k = 0
    return (bar, (use & 1) ^ 1, use)


def run(roles, seed, max_steps=3_000_000):
    """roles: name -> generator.  A generator yields a (barrier, parity, need) wait, or None to
    give up its turn; everything else it does between yields is atomic."""
    rng = random.Random(seed)
    live = dict(roles)
    blocked = {}
    idle_sweeps = 0
    for _ in range(max_steps):
        if not live:
            return
        name = rng.choice(list(live))
        if name in blocked:
            bar, parity, need = blocked[name]
            if not bar.poll(parity, need):
                idle_sweeps += 1
                if idle_sweeps > 50 * len(live) and all(
                        n in blocked and not blocked[n][0].poll(blocked[n][1], blocked[n][2]) for n in live):
                    raise ProtocolError(f"deadlock: { {n: blocked[n][0].name for n in live} }")
                continue
            del blocked[name]
        idle_sweeps = 0
        try:
            op = next(live[name])
        except StopIteration:
            del live[name]
            continue
        if op is not None:
            blocked[name] = op
    raise ProtocolError("simulation did not finish")


def tma_engine(in_flight, total, seed):
    """Completes issued loads in random order, at random later times."""
    rng = random.Random(seed)
    done = 0
    while done < total:
        if in_flight and rng.random() < 0.5:
            bar, n = in_flight.pop(rng.randrange(len(in_flight)))
            bar.complete_tx(n)
            done += 1
        yield None


def rounds_of_group(rounds, stages, groups, group, by_stage):
    if by_stage:
        return [i for i in range(rounds) if (i % stages) % groups == group]
    return list(range(group, rounds, groups))


# ---------------------------------------------------------------------------------------
# single-CTA kernel (gemm_tcgen05.cu):
#   full[s]   count 1 + bytes : producer's expect_tx, TMA completes        -> converters, MMA issuer
#   aready[s] count 4         : one arrive per converter warp of the group -> MMA issuer
#   empty[s]  count 1         : tcgen05.commit after the stage's MMAs      -> producer
#   accfull   count 1         : tcgen05.commit after the last stage        -> epilogue (all converter warps)
# ---------------------------------------------------------------------------------------
def single_cta(rounds, stages, groups, by_stage=True, seed=0):
    full = [Barrier(f"full{s}", 1) for s in range(stages)]
    aready = [Barrier(f"aready{s}", 4) for s in range(stages)]
    empty = [Barrier(f"empty{s}", 1) for s in range(stages)]
    acc = Barrier("accfull", 1)
    in_flight = []

    def producer():
        for i in range(rounds):
            s, k = i % stages, i // stages
            yield producer_wait(empty[s], k)
            full[s].arrive(tx=1000)
            in_flight.append((full[s], 1000))

    def mma():
        for i in range(rounds):
            s, k = i % stages, i // stages
            yield consumer_wait(aready[s], k)
            yield consumer_wait(full[s], k)
            empty[s].arrive()
        acc.arrive()

    def converter(group):
        for i in rounds_of_group(rounds, stages, groups, group, by_stage):
            s, k = i % stages, i // stages
            yield consumer_wait(full[s], k)
            yield None                      # the conversion itself takes time
            aready[s].arrive()
        yield consumer_wait(acc, 0)

    roles = {"producer": producer(), "tma": tma_engine(in_flight, rounds, seed), "mma": mma()}
    for g in range(groups):
        for w in range(4):
            roles[f"conv{g}.{w}"] = converter(g)
    return roles


# the (stages, groups) pairs the kernel is instantiated with: 5 stages at 256 tokens per tile,
# 4 at 128, 6 at 64, 7 at 32 and 16; 1 to 3 converter groups
SINGLE = [(5, 3), (4, 3), (6, 3), (7, 3), (5, 2), (4, 2), (7, 2), (5, 1), (7, 1)]


@pytest.mark.parametrize("stages,groups", SINGLE)
@pytest.mark.parametrize("rounds", [1, 2, 3, 8, 43, 172])
def test_single_cta_protocol(rounds, stages, groups):
    for seed in range(6):
        run(single_cta(rounds, stages, groups, seed=seed), seed)


def test_round_robin_groups_are_ambiguous():
    # rounds dealt round-robin over 3 groups with 4 or 5 stages: some schedule with out-of-order
    # TMA completion makes a converter poll a stage whose previous phase is still open
    for stages in (4, 5):
        with pytest.raises(ProtocolError, match="ambiguous"):
            for seed in range(300):
                run(single_cta(40, stages, 3, by_stage=False, seed=seed), seed)


def test_round_robin_is_fine_when_groups_divide_stages():
    for seed in range(20):
        run(single_cta(40, 6, 3, by_stage=False, seed=seed), seed)


# ---------------------------------------------------------------------------------------
# CTA pair (gemm_tcgen05_2cta.cu); rank 0 is the leader:
#   wfull[s]  each CTA, count 1 + bytes : this CTA's codes                                -> its converters
#   xfull[s]  leader,   count 1 + bytes : the activation halves of BOTH CTAs              -> MMA issuer
#   aready[s] leader,   count 8         : 4 converter warps x 2 CTAs (remote arrive)      -> MMA issuer
#   empty[s]  each CTA, count 1         : one commit per CTA's barrier                     -> its producer
#   accfull   each CTA, count 1         : the same pair of commits after the last stage    -> its epilogue
# ---------------------------------------------------------------------------------------
def cta_pair(rounds, stages=4, groups=3, by_stage=True, aready_count=8, seed=0):
    wfull = [[Barrier(f"wfull{r}.{s}", 1) for s in range(stages)] for r in range(2)]
    xfull = [Barrier(f"xfull{s}", 1) for s in range(stages)]
    aready = [Barrier(f"aready{s}", aready_count) for s in range(stages)]
    empty = [[Barrier(f"empty{r}.{s}", 1) for s in range(stages)] for r in range(2)]
    acc = [Barrier(f"acc{r}", 1) for r in range(2)]
    in_flight = []

    def producer(rank):
        for i in range(rounds):
            s, k = i % stages, i // stages
            yield producer_wait(empty[rank][s], k)
            wfull[rank][s].arrive(tx=100)
            if rank == 0:
                xfull[s].arrive(tx=2 * 300)   # the leader expects both halves
            in_flight.append((wfull[rank][s], 100))
            in_flight.append((xfull[s], 300))  # either CTA's half completes on the leader's barrier

    def mma_leader():
        for i in range(rounds):
            s, k = i % stages, i // stages
            yield consumer_wait(aready[s], k)
            yield consumer_wait(xfull[s], k)
            empty[0][s].arrive()
            empty[1][s].arrive()
        acc[0].arrive()
        acc[1].arrive()

    def converter(rank, group):
        for i in rounds_of_group(rounds, stages, groups, group, by_stage):
            s, k = i % stages, i // stages
            yield consumer_wait(wfull[rank][s], k)
            yield None
            aready[s].arrive()
        yield consumer_wait(acc[rank], 0)

    roles = {"tma": tma_engine(in_flight, 4 * rounds, seed), "mma": mma_leader()}
    for r in range(2):
        roles[f"producer{r}"] = producer(r)
        for g in range(groups):
            for w in range(4):
                roles[f"conv{r}.{g}.{w}"] = converter(r, g)
    return roles


@pytest.mark.parametrize("rounds", [1, 2, 3, 4, 5, 9, 32, 86])
def test_cta_pair_protocol(rounds):
    for seed in range(6):
        run(cta_pair(rounds, seed=seed), seed)


def test_model_catches_a_wrong_arrival_count():
    with pytest.raises(ProtocolError):
        for seed in range(20):
            run(cta_pair(8, aready_count=4, seed=seed), seed)


def test_model_catches_a_missing_release():
    # a producer that waits on a barrier nobody arrives on: reported as a deadlock, not a hang
    lonely = Barrier("never", 1)

    def waiter():
        yield consumer_wait(lonely, 0)

    with pytest.raises(ProtocolError, match="deadlock"):
        run({"w": waiter()}, 0)
