"""The mbarrier protocol of the CTA-pair GEMM kernel (csrc/gemm_tc2.cu), modelled on CPU.

The kernel's three roles - TMA producer (both CTAs), MMA issuer (leader) and 2 x 8 epilogue warps - are
restated as Python generators that perform the same barrier operations in the same order as the CUDA code,
for the kernel's tile shape (one 256x512 tile owns both tensor-memory halves, half 1 trails half 0 by `skew`
k-blocks) and for the 256x256 shape that was measured against it and dropped from the kernel (consecutive tiles
alternate between the halves; kept here because the model is the record of why that protocol is sound).  Asynchronous
completions (TMA bytes landing, tcgen05.commit arrivals) are delivered at random later times.  A random
scheduler interleaves everything and the model checks
  * liveness: every role finishes (no wait that nothing satisfies),
  * shared-memory ring: a stage is refilled only after the MMAs that read it have completed, and is read only
    after both CTAs' loads of it have landed,
  * tensor memory: a half is overwritten only after all 16 epilogue warps have drained the previous tile in
    it, and is drained only after its last MMA has completed,
  * every tile is stored exactly once by every epilogue warp.
This is a model of the protocol, not of the arithmetic; the GPU tests cover the results."""

import random

import pytest

SCHED_SLOTS = 4
EPI_WARPS = 8


class Barrier:
    def __init__(self, count):
        self.count, self.pending, self.tx, self.phase = count, count, 0, 0

    def _check(self):
        if self.pending == 0 and self.tx == 0:
            self.phase += 1
            self.pending = self.count

    def arrive(self):
        assert self.pending > 0, "more arrivals than the barrier expects in one phase"
        self.pending -= 1
        self._check()

    def arrive_expect_tx(self, nbytes):
        self.tx += nbytes
        self.arrive()

    def complete_tx(self, nbytes):
        self.tx -= nbytes
        self._check()

    def passed(self, parity):
        return (self.phase & 1) != parity


class Cta:
    def __init__(self, stages):
        self.full = [Barrier(1) for _ in range(stages)]
        self.empty = [Barrier(1) for _ in range(stages)]
        self.acc_full = [Barrier(1) for _ in range(2)]
        self.acc_empty = [Barrier(2 * EPI_WARPS) for _ in range(2)]
        self.sched_full = [Barrier(1) for _ in range(SCHED_SLOTS)]
        self.sched_empty = [Barrier(2 + 2 * EPI_WARPS) for _ in range(SCHED_SLOTS)]
        self.sched_tile = [None] * SCHED_SLOTS


class Model:
    def __init__(self, tiles, halves_mode, stages, skew, n_pairs, seed):
        self.tiles, self.HALVES, self.STAGES, self.skew_param = tiles, halves_mode, stages, skew
        self.rng = random.Random(seed)
        self.cta = [Cta(stages), Cta(stages)]  # leader, peer
        self.n_pairs = n_pairs  # other pairs also draw from the counter: this pair sees every n-th tile or so
        self.next_tile = 0
        self.async_ops = []  # deferred completions: (fifo key or None, callable)
        # ground truth for the hazard checks
        self.stage_loaded = [[False, False] for _ in range(stages)]  # per stage: [leader's loads, peer's loads] landed
        self.stage_readers = [0] * stages  # MMAs issued on the stage whose completion has not been observed
        self.acc_state = ["free", "free"]  # free -> accumulating -> complete -> (16 drains) -> free
        self.acc_drains = [0, 0]
        self.acc_tile = [None, None]
        self.stored = {}

    # ---- asynchronous completions ----------------------------------------------------------------
    def defer(self, fn, fifo=None):
        self.async_ops.append((fifo, fn))

    def deliver_one(self):
        """Delivers one deferred completion; commits of the MMA thread complete in issue order."""
        candidates = []
        seen_fifo = set()
        for i, (fifo, _) in enumerate(self.async_ops):
            if fifo is None:
                candidates.append(i)
            elif fifo not in seen_fifo:
                seen_fifo.add(fifo)
                candidates.append(i)
        i = self.rng.choice(candidates)
        _, fn = self.async_ops.pop(i)
        fn()

    # ---- tile bookkeeping ------------------------------------------------------------------------
    def draw(self):
        """Leader's producer draws the next tile of this pair (dynamic counter shared with other pairs)."""
        while self.next_tile < len(self.tiles) and self.rng.random() < 1 - 1 / self.n_pairs:
            self.next_tile += 1  # taken by another pair
        t = self.next_tile
        self.next_tile += 1
        return t if t < len(self.tiles) else -1

    # ---- roles (generators yield a predicate they wait for) ------------------------------------------
    def producer(self, rank):
        me, leader = self.cta[rank], self.cta[0]
        stage, phase, sslot, sphase = 0, 0, 0, 0
        tile = self.draw() if rank == 0 else None
        while True:
            nxt = -1
            if rank == 0:
                bar = leader.sched_empty[sslot]
                yield lambda bar=bar, p=sphase ^ 1: bar.passed(p)
                v = tile
                for c in self.cta:
                    c.sched_tile[sslot] = v
                    c.sched_full[sslot].arrive()
                if v >= 0:
                    nxt = self.draw()
            else:
                bar = me.sched_full[sslot]
                yield lambda bar=bar, p=sphase: bar.passed(p)
                tile = me.sched_tile[sslot]
                leader.sched_empty[sslot].arrive()
            sslot += 1
            if sslot == SCHED_SLOTS:
                sslot, sphase = 0, sphase ^ 1
            if tile < 0:
                return
            nkb, halves, valid = self.tiles[tile]
            if valid:
                for _ in range(nkb):
                    bar = me.empty[stage]
                    yield lambda bar=bar, p=phase ^ 1: bar.passed(p)
                    assert self.stage_readers[stage] == 0, "ring stage refilled while MMAs still read it"
                    self.stage_loaded[stage][rank] = False
                    nbytes = 1 + halves  # A slab + one B slab per half, in slab units
                    if rank == 0:
                        leader.full[stage].arrive_expect_tx(2 * nbytes)

                    def land(stage=stage, rank=rank, nbytes=nbytes):
                        self.stage_loaded[stage][rank] = True
                        leader.full[stage].complete_tx(nbytes)

                    self.defer(land)
                    stage += 1
                    if stage == self.STAGES:
                        stage, phase = 0, phase ^ 1
            if rank == 0:
                tile = nxt

    def commit_pair(self, which, index, extra=None):
        """tcgen05.commit on the barrier `which[index]` of both CTAs: arrives once prior MMAs have completed."""

        def done():
            if extra:
                extra()
            for c in self.cta:
                getattr(c, which)[index].arrive()

        self.defer(done, fifo="mma")

    def mma(self):
        leader = self.cta[0]
        stage, phase, acc_phase, tile_count, sslot, sphase = 0, 0, 0, 0, 0, 0
        while True:
            bar = leader.sched_full[sslot]
            yield lambda bar=bar, p=sphase: bar.passed(p)
            tile = leader.sched_tile[sslot]
            leader.sched_empty[sslot].arrive()
            sslot += 1
            if sslot == SCHED_SLOTS:
                sslot, sphase = 0, sphase ^ 1
            if tile < 0:
                return
            nkb, halves, valid = self.tiles[tile]
            if not valid:
                continue
            h0 = (tile_count & 1) if self.HALVES == 1 else 0
            ph0 = ((tile_count >> 1) & 1) if self.HALVES == 1 else acc_phase
            skew = min(self.skew_param, nkb) if halves == 2 else 0

            def begin(h, tile=tile):
                assert self.acc_state[h] == "free", f"tensor-memory half {h} overwritten before it was drained"
                self.acc_state[h], self.acc_tile[h], self.acc_drains[h] = "accumulating", tile, 0

            def issue(st):
                assert all(self.stage_loaded[st]), "MMA reads a ring stage whose loads have not landed"
                self.stage_readers[st] += 1

            def complete(h):
                def fn():
                    assert self.acc_state[h] == "accumulating"
                    self.acc_state[h] = "complete"

                return fn

            for step in range(nkb + skew):
                if step < nkb:
                    bar = leader.full[stage]
                    yield lambda bar=bar, p=phase: bar.passed(p)
                    if step == 0:
                        bar = leader.acc_empty[h0]
                        yield lambda bar=bar, p=ph0 ^ 1: bar.passed(p)
                        begin(h0)
                    issue(stage)
                    if step == nkb - 1:
                        self.commit_pair("acc_full", h0, extra=complete(h0))
                kb1 = step - skew
                if kb1 >= 0:
                    behind = skew if step < nkb else nkb - kb1
                    st1 = (stage + self.STAGES - behind) % self.STAGES
                    if halves == 2:
                        if kb1 == 0:
                            bar = leader.acc_empty[1]
                            yield lambda bar=bar, p=acc_phase ^ 1: bar.passed(p)
                            begin(1)
                        issue(st1)
                    readers = 2 if halves == 2 else 1

                    def release(st1=st1, readers=readers):
                        self.stage_readers[st1] -= readers

                    self.commit_pair("empty", st1, extra=release)
                if step < nkb:
                    stage += 1
                    if stage == self.STAGES:
                        stage, phase = 0, phase ^ 1
            if nkb > 0:
                if halves == 2:
                    self.commit_pair("acc_full", 1, extra=complete(1))
            else:
                for h in range(halves):
                    hb = h0 if self.HALVES == 1 else h
                    phb = ph0 if self.HALVES == 1 else acc_phase
                    bar = leader.acc_empty[hb]
                    yield lambda bar=bar, p=phb ^ 1: bar.passed(p)
                    begin(hb)
                    self.acc_state[hb] = "complete"
                    for c in self.cta:
                        c.acc_full[hb].arrive()
            if self.HALVES == 2 and halves == 1:
                bar = leader.acc_empty[1]
                yield lambda bar=bar, p=acc_phase ^ 1: bar.passed(p)
                begin(1)
                self.acc_state[1] = "complete"
                for c in self.cta:
                    c.acc_full[1].arrive()
            acc_phase ^= 1
            tile_count += 1

    def epilogue(self, rank, warp):
        me, leader = self.cta[rank], self.cta[0]
        acc_phase, tile_count, sslot, sphase = 0, 0, 0, 0
        while True:
            bar = me.sched_full[sslot]
            yield lambda bar=bar, p=sphase: bar.passed(p)
            tile = me.sched_tile[sslot]
            leader.sched_empty[sslot].arrive()
            sslot += 1
            if sslot == SCHED_SLOTS:
                sslot, sphase = 0, sphase ^ 1
            if tile < 0:
                return
            nkb, halves, valid = self.tiles[tile]
            if not valid:
                continue
            for h in range(self.HALVES):
                hs = (tile_count & 1) if self.HALVES == 1 else h
                phs = ((tile_count >> 1) & 1) if self.HALVES == 1 else acc_phase
                bar = me.acc_full[hs]
                yield lambda bar=bar, p=phs: bar.passed(p)
                assert self.acc_state[hs] == "complete" and self.acc_tile[hs] == tile, "epilogue reads a half that is not ready"
                key = (tile, h, rank, warp)
                assert key not in self.stored
                self.stored[key] = True
                yield lambda: True  # the stores take a while; others run meanwhile
                self.acc_drains[hs] += 1
                if self.acc_drains[hs] == 2 * EPI_WARPS:
                    self.acc_state[hs] = "free"
                leader.acc_empty[hs].arrive()
            acc_phase ^= 1
            tile_count += 1

    # ---- scheduler ---------------------------------------------------------------------------------
    def run(self):
        roles = {"producer0": self.producer(0), "producer1": self.producer(1), "mma": self.mma()}
        for r in range(2):
            for w in range(EPI_WARPS):
                roles[f"epilogue{r}.{w}"] = self.epilogue(r, w)
        waiting = {}
        for name, gen in list(roles.items()):
            try:
                waiting[name] = next(gen)
            except StopIteration:
                del roles[name]
        steps = 0
        while roles or self.async_ops:
            steps += 1
            assert steps < 2_000_000
            runnable = [n for n in roles if waiting[n]()]
            choices = runnable + (["<async>"] if self.async_ops else [])
            assert choices, f"deadlock: {sorted(roles)} wait and nothing is in flight"
            pick = self.rng.choice(choices)
            if pick == "<async>":
                self.deliver_one()
                continue
            try:
                waiting[pick] = next(roles[pick])
            except StopIteration:
                del roles[pick], waiting[pick]


def _tiles(rng, n, halves_mode, max_kb):
    out = []
    for _ in range(n):
        nkb = rng.choice([0, 1, 2, 3, max_kb, rng.randint(1, max_kb)])
        halves = 2 if halves_mode == 2 and rng.random() < 0.7 else 1
        out.append((nkb, halves, rng.random() > 0.1))  # a tenth of the tiles lie beyond the used rows
    return out


@pytest.mark.parametrize("halves_mode,stages", [(2, 4), (1, 6)])
@pytest.mark.parametrize("skew", [0, 1, 2])
@pytest.mark.parametrize("seed", range(6))
def test_pair_kernel_protocol(halves_mode, stages, skew, seed):
    if halves_mode == 1 and skew:
        pytest.skip("the skew only exists for tiles with two halves")
    rng = random.Random(1000 * halves_mode + 10 * skew + seed)
    tiles = _tiles(rng, 60, halves_mode, max_kb=9)
    model = Model(tiles, halves_mode, stages, skew, n_pairs=rng.choice([1, 2, 5]), seed=seed)
    model.run()
    # every valid tile this pair drew was stored by all 16 warps for each half the epilogue walks
    drawn = {key[0] for key in model.stored}
    for tile in drawn:
        for h in range(halves_mode):
            for rank in range(2):
                for warp in range(EPI_WARPS):
                    assert (tile, h, rank, warp) in model.stored
    assert all(s == "free" for s in model.acc_state) and not any(model.stage_readers)
