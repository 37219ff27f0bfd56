"""Host-side protocol checker for the sm_100a GEMM pipeline.

The reference crate race-checks its kernels by running them in a CPU
simulator with per-byte shared-memory metadata, per-warp vector clocks and an
mbarrier phase/transaction model (src/sim/exec.rs:35-53, 98-151, 870-1011,
1545-1740, 1886-1922).  The hand-written tcgen05 kernel cannot run in that
simulator, so this module restates the kernel's synchronisation protocol -
who waits on, arrives on and commits to which mbarrier, and which agent reads
or writes which shared-memory stage and TMEM half - and checks it with the
same rules:

* agents (producer thread, MMA-issuing thread, epilogue warps, and the two
  asynchronous agents: the TMA unit and the tensor core) carry vector clocks;
* a read of a resource must happen after its last write, a write after every
  earlier read and write (read-after-write, write-after-read, write-after-write);
* an mbarrier phase completes when its arrival count and its transaction count
  both reach zero; a successful wait acquires everything released into that
  phase; more bytes than expected, or a phase that completes while a copy that
  reports to it is still uncounted, is an error;
* the parity rule: a wait for phase n must succeed exactly when n + 1 phases
  have completed; if the hardware test `completed % 2 != parity` would pass
  with any other count, the parity aliases an older or newer phase
  (src/sim/exec.rs:1648-1668);
* nothing may be left blocked at the end (the simulator reports loops that do
  not terminate; here: deadlock).

The several-destination form of the kernel adds a pusher thread per CTA: the
epilogue warps store their part of a tile to C and publish their own tile
count in a shared-memory slot (release), the pusher waits until every warp's
slot has reached the tile (acquire),
lets the TMA unit load the tile from C into one of two staging buffers
(reported to an mbarrier), issues the bulk stores that read the buffer, and
waits for the stores of the previous chunk to have read theirs before the
buffer is filled again.  The counter, the bulk groups and the global-memory
tile parts are modelled with the same clocks.

`gemm_schedule` generates the per-agent programs of `gemm_tn_kernel` for a
tiling (CTA group, ring stages, accumulator halves and buffers) and a list of
work units; `mutations` name deliberate protocol bugs used by the tests to show
that the checker sees them.  It checks the protocol, not the CUDA source.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field


class ProtocolError(Exception):
    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


# ---- vector clocks -------------------------------------------------------------
class Clock(dict):
    def join(self, other: "Clock") -> None:
        for a, t in other.items():
            if self.get(a, 0) < t:
                self[a] = t

    def knows(self, stamp) -> bool:
        agent, tick = stamp
        return self.get(agent, 0) >= tick

    def copy(self) -> "Clock":
        return Clock(self)


@dataclass
class Barrier:
    name: str
    count: int                      # arrivals per phase
    pending: int = 0                # arrivals left in the current phase
    tx: int = 0                     # bytes expected minus bytes landed
    completed: int = 0              # phases completed so far
    release: Clock = field(default_factory=Clock)
    phase_clock: dict = field(default_factory=dict)  # phase index -> clock released into it

    def __post_init__(self):
        self.pending = self.count

    def _maybe_complete(self):
        if self.pending == 0 and self.tx == 0:
            self.phase_clock[self.completed] = self.release
            self.completed += 1
            self.release = Clock()
            self.pending = self.count
        elif self.pending == 0 and self.tx < 0:
            raise ProtocolError("tx", f"{self.name}: more bytes landed than expect_tx announced")

    def arrive(self, clock: Clock, expect: int = 0):
        if self.pending == 0:
            raise ProtocolError("arrive", f"{self.name}: more arrivals than the barrier was initialised for")
        self.tx += expect
        self.release.join(clock)
        self.pending -= 1
        self._maybe_complete()

    def complete_tx(self, clock: Clock, nbytes: int):
        self.tx -= nbytes
        self.release.join(clock)
        self._maybe_complete()


@dataclass
class Resource:
    name: str
    write: tuple = None             # stamp (agent, tick) of the last write
    reads: list = field(default_factory=list)


class Machine:
    def __init__(self):
        self.clocks = {}
        self.barriers = {}
        self.resources = {}
        self.counters = {}   # name -> [value, clock released into it]
        self.groups = {}     # issuing agent -> list of bulk groups (each a clock of the reads it still does)

    def clock(self, agent) -> Clock:
        return self.clocks.setdefault(agent, Clock())

    def tick(self, agent):
        c = self.clock(agent)
        c[agent] = c.get(agent, 0) + 1
        return (agent, c[agent])

    def res(self, name) -> Resource:
        return self.resources.setdefault(name, Resource(name))

    # An access by `agent`, ordered after everything `after` (a clock) knows.
    def write(self, agent, name, after: Clock):
        c = self.clock(agent)
        c.join(after)
        r = self.res(name)
        if r.write and not c.knows(r.write):
            raise ProtocolError("race", f"{agent} writes {name} without being ordered after the write by {r.write[0]}")
        for rd in r.reads:
            if not c.knows(rd):
                raise ProtocolError("race", f"{agent} overwrites {name} while {rd[0]} may still be reading it")
        r.write, r.reads = self.tick(agent), []

    def read(self, agent, name, after: Clock):
        c = self.clock(agent)
        c.join(after)
        r = self.res(name)
        if r.write is None:
            raise ProtocolError("uninitialised", f"{agent} reads {name} before anything wrote it")
        if not c.knows(r.write):
            raise ProtocolError("race", f"{agent} reads {name} without being ordered after the write by {r.write[0]}")
        r.reads.append(self.tick(agent))

    def accumulate(self, agent, name, after: Clock, first: bool):
        """Read-modify-write by the tensor core; `first` overwrites (accumulate flag 0)."""
        if first:
            self.write(agent, name, after)
        else:
            self.read(agent, name, after)
            r = self.res(name)
            r.write, r.reads = self.tick(agent), []


# ---- programs --------------------------------------------------------------------
# An op is a tuple; the first element names it:
#   ("wait", barrier, phase)                 block until `phase` of the barrier completed, acquire it
#   ("arrive", barrier) / ("expect", barrier, bytes)   arrive (with expect_tx)
#   ("tma", cta, stage, bytes, barrier)      TMA writes the stage, bytes reported to barrier
#   ("mma", [stage resources], [tmem resources], first)
#   ("commit", barrier)                      arrival by the tensor core after all MMAs issued so far
#   ("ld", tmem resource)                    epilogue warp reads a TMEM half
#   ("st", resource)                         epilogue warp writes its part of a tile of C
#   ("signal", counter)                      release-increment of a shared-memory counter
#   ("wait_count", counter, value)           acquire-poll until the counter has reached value
#   ("tma_load", cta, [C parts], buffer, bytes, barrier)   TMA reads the parts, writes the staging buffer
#   ("tma_store", cta, buffer)               TMA reads the staging buffer (one bulk group per op)
#   ("wait_read", keep)                      all but the newest `keep` bulk groups have read their source
#   ("tma_store", cta, buffer, destination)  ... a store that also names what it writes (another GPU's rows of C)
#   ("wait_all",)                            every bulk group of the thread is complete, its writes included
def run(programs: dict, barriers: dict, seed: int = 0, tma_bytes_to=None, max_burst: int = 0, stalls=None) -> Machine:
    """Interleave the agents' programs: in every round each agent, in random order, runs until it
    blocks, or for a random number of steps up to `max_burst` when that is set (finer interleavings).
    `stalls` maps an agent to (program counter, rounds): the agent pauses that many rounds before that
    operation - a warp that the hardware scheduler leaves waiting while the others run on."""
    stalls = {a: list(v) for a, v in (stalls or {}).items()}
    m = Machine()
    m.barriers = {n: Barrier(n, c) for n, c in barriers.items()}
    pcs = {a: 0 for a in programs}
    rng = random.Random(seed)
    agents = list(programs)
    while True:
        progressed, done = False, True
        rng.shuffle(agents)
        for a in agents:
            prog = programs[a]
            budget = rng.randint(1, max_burst) if max_burst else -1
            while pcs[a] < len(prog):
                done = False
                if budget == 0:
                    break
                budget -= 1
                if a in stalls and stalls[a][0] == pcs[a] and stalls[a][1] > 0:
                    stalls[a][1] -= 1
                    progressed = True
                    break
                op = prog[pcs[a]]
                kind = op[0]
                if kind == "wait":
                    bar, phase = m.barriers[op[1]], op[2]
                    if (bar.completed % 2) == (phase % 2):
                        break  # the hardware test `completed % 2 != parity` fails: still blocked
                    if bar.completed != phase + 1:
                        raise ProtocolError("parity", f"{a} waits for phase {phase} of {op[1]} (parity {phase % 2}); the "
                                                      f"test passes with {bar.completed} phases completed")
                    if phase >= 0:
                        m.clock(a).join(bar.phase_clock[phase])
                elif kind == "arrive":
                    m.tick(a)
                    m.barriers[op[1]].arrive(m.clock(a))
                elif kind == "expect":
                    m.tick(a)
                    m.barriers[op[1]].arrive(m.clock(a), expect=op[2])
                elif kind == "tma":
                    _, cta, stage, nbytes, bar = op
                    agent = f"tma{cta}"
                    m.write(agent, f"smem{cta}.{stage}", m.clock(a))
                    m.barriers[bar].complete_tx(m.clock(agent), nbytes)
                elif kind == "mma":
                    _, stages, tmems, first = op
                    for s in stages:
                        m.read("umma", s, m.clock(a))
                    for t in tmems:
                        m.accumulate("umma", t, m.clock(a), first)
                elif kind == "commit":
                    m.clock("umma").join(m.clock(a))
                    m.barriers[op[1]].arrive(m.clock("umma"))
                elif kind == "ld":
                    m.read(a, op[1], m.clock(a))
                elif kind == "st":
                    m.write(a, op[1], m.clock(a))
                elif kind == "signal":
                    m.tick(a)
                    ctr = m.counters.setdefault(op[1], [0, Clock()])
                    ctr[0] += 1
                    ctr[1].join(m.clock(a))
                elif kind == "wait_count":
                    ctr = m.counters.setdefault(op[1], [0, Clock()])
                    if ctr[0] < op[2]:
                        break
                    m.clock(a).join(ctr[1])
                elif kind == "tma_load":
                    # Every bulk copy is an asynchronous agent of its own: copies are ordered after the
                    # thread that issued them, not after one another.
                    _, cta, parts, buf, nbytes, bar = op
                    agent = f"tma_load{cta}.{pcs[a]}"
                    for part in parts:
                        m.read(agent, part, m.clock(a))
                    m.write(agent, buf, m.clock(a))
                    m.barriers[bar].complete_tx(m.clock(agent), nbytes)
                elif kind == "tma_store":
                    cta, buf = op[1], op[2]
                    agent = f"tma_store{cta}.{pcs[a]}"
                    m.read(agent, buf, m.clock(a))
                    if len(op) > 3:  # the destination in another GPU's memory, written by the same copy
                        m.write(agent, op[3], m.clock(a))
                    m.groups.setdefault(a, []).append(m.clock(agent).copy())
                elif kind == "wait_all":  # cp.async.bulk.wait_group 0: reads and writes of every group are complete
                    for g in m.groups.get(a, []):
                        m.clock(a).join(g)
                elif kind == "wait_read":
                    groups = m.groups.get(a, [])
                    for g in groups[:len(groups) - op[1]]:
                        m.clock(a).join(g)
                else:
                    raise ValueError(op)
                pcs[a] += 1
                progressed = True
        if done:
            break
        if not progressed:
            stuck = {a: programs[a][pcs[a]] for a in agents if pcs[a] < len(programs[a])}
            raise ProtocolError("deadlock", f"no agent can proceed: {stuck}")
    for b in m.barriers.values():
        if b.tx != 0:
            raise ProtocolError("tx", f"{b.name}: {b.tx} bytes still expected at the end (expect_tx too large or a copy missing)")
    return m


# ---- the GEMM kernel's protocol ------------------------------------------------------
def gemm_schedule(cta_group: int = 2, stages: int = 4, mh: int = 2, acc_bufs: int = 1, units=(8, 8, 8),
                  stage_bytes: int = 48 * 1024, mutations=(), push_chunks: int = 0, epilogue_warps: int = 8,
                  tmem_empty_arrivals: int = None, expect_tx: int = None, push_bytes: int = 16 * 1024, kps: int = 1):
    """Programs and barriers of gemm_tn_kernel for one cluster.

    `units` lists the k-block count of each work unit the cluster processes (0 =
    an empty k range).  `kps` k blocks share one ring stage (one full/empty
    barrier pair; the last stage of a unit may hold fewer); `stage_bytes` are the
    bytes of ONE k block in one CTA, `expect_tx` what the leader announces per k
    block.  `tmem_empty_arrivals` (count the accumulator-free barriers
    are initialised with) and `expect_tx` (bytes the leader announces per stage)
    default to what the schedule itself implies - one arrival per epilogue warp of
    the group, every CTA's stage bytes; `tiling_from_library` passes the values the
    compiled kernel uses instead, so that a kernel whose constants disagree with its
    own schedule fails here.  Mutations (protocol bugs for the tests):
      "producer_skips_empty_wait"  the producer refills a stage without waiting for its release
      "mma_skips_full_wait"        the MMA issuer does not wait for the loads
      "mma_skips_tmem_wait"        ... nor for the epilogue to drain the accumulator
      "epilogue_arrives_early"     a warp hands the TMEM half back before reading it
      "expect_tx_short"            the leader announces one CTA's bytes instead of the group's
      "wrong_empty_parity"         the producer starts with the parity of a full ring
      "no_peer_commit"             the leader forgets to release the peer CTA's stages
    With push_chunks > 0 every CTA also runs the pusher (that many chunks per tile):
      "epilogue_signals_early"     a warp counts itself in before it has stored its part of the tile
      "pusher_skips_tile_wait"     the pusher loads a tile without waiting for the warps' count
      "pusher_skips_load_wait"     ... issues the stores without waiting for the load to land
      "pusher_skips_read_wait"     ... refills a staging buffer that a store may still be reading
      "pusher_wrong_parity"        ... waits on the load barrier with the parity of the other buffer's use
      "shared_tile_counter"        the warps add to one shared count instead of publishing a slot each: a warp
                                   that runs a tile ahead is then counted for one that has not stored yet
    """
    mut = set(mutations)
    ctas = range(cta_group)
    barriers = {}
    for s in range(stages):
        barriers[f"full.{s}"] = 1  # on the leader; counts the bytes of the whole group
        for c in ctas:
            barriers[f"empty{c}.{s}"] = 1
    for b in range(acc_bufs):
        for c in ctas:
            barriers[f"tfull{c}.{b}"] = 1
        for h in range(mh):
            # one arrival per epilogue warp of the group, unless the caller says what the kernel uses
            barriers[f"tempty.{b}.{h}"] = tmem_empty_arrivals if tmem_empty_arrivals is not None else epilogue_warps * cta_group
    programs = {f"producer{c}": [] for c in ctas}
    programs["mma"] = []
    for c in ctas:
        for w in range(epilogue_warps):
            programs[f"epilogue{c}.{w}"] = []

    if push_chunks:
        for c in ctas:
            barriers[f"push{c}.0"] = 1
            barriers[f"push{c}.1"] = 1
            programs[f"pusher{c}"] = []
    pushed = 0  # chunks pushed so far per CTA
    fill = 0   # ring slots filled so far (same sequence in every role)
    it = 0     # non-empty units so far
    for kbs in units:
        buf, use = it % acc_bufs, it // acc_bufs
        for kb0 in range(0, kbs, kps):
            nk = min(kps, kbs - kb0)
            s, rnd = fill % stages, fill // stages
            for c in ctas:
                p = programs[f"producer{c}"]
                if "producer_skips_empty_wait" not in mut:
                    p.append(("wait", f"empty{c}.{s}", rnd - 1 + (1 if "wrong_empty_parity" in mut else 0)))
                if c == 0:
                    per_kb = stage_bytes if "expect_tx_short" in mut else (expect_tx if expect_tx is not None else stage_bytes * cta_group)
                    p.append(("expect", f"full.{s}", nk * per_kb))
                p.append(("tma", c, s, nk * stage_bytes, f"full.{s}"))
            mma = programs["mma"]
            if "mma_skips_full_wait" not in mut:
                mma.append(("wait", f"full.{s}", rnd))
            for kb in range(kb0, kb0 + nk):
                for h in range(mh):
                    if kb == 0 and "mma_skips_tmem_wait" not in mut:
                        mma.append(("wait", f"tempty.{buf}.{h}", use - 1))
                    mma.append(("mma", [f"smem{c}.{s}" for c in ctas], [f"tmem{c}.{buf}.{h}" for c in ctas], kb == 0))
            for c in ctas:
                if c == 0 or "no_peer_commit" not in mut:
                    mma.append(("commit", f"empty{c}.{s}"))
            fill += 1
        if kbs > 0:
            for c in ctas:
                programs["mma"].append(("commit", f"tfull{c}.{buf}"))
            for c in ctas:
                for w in range(epilogue_warps):
                    e = programs[f"epilogue{c}.{w}"]
                    e.append(("wait", f"tfull{c}.{buf}", use))
                    for h in range(mh):
                        if "epilogue_arrives_early" in mut:
                            e.append(("arrive", f"tempty.{buf}.{h}"))
                        e.append(("ld", f"tmem{c}.{buf}.{h}"))
                        if "epilogue_arrives_early" not in mut:
                            e.append(("arrive", f"tempty.{buf}.{h}"))
                    if push_chunks:
                        slot = f"stored{c}" if "shared_tile_counter" in mut else f"stored{c}.{w}"
                        if "epilogue_signals_early" in mut:
                            e.append(("signal", slot))
                        e.append(("st", f"c{c}.{it}.{w}"))
                        if "epilogue_signals_early" not in mut:
                            e.append(("signal", slot))
            if push_chunks:
                # The load of a chunk is issued one iteration ahead of its stores, after the stores of
                # the chunk before have read the buffer it fills (the kernel's loop, unrolled).
                for c in ctas:
                    p = programs[f"pusher{c}"]
                    parts = [f"c{c}.{it}.{w}" for w in range(epilogue_warps)]
                    for ch in range(push_chunks):
                        g = pushed + ch
                        if ch == 0 and "pusher_skips_tile_wait" not in mut:
                            if "shared_tile_counter" in mut:
                                p.append(("wait_count", f"stored{c}", epilogue_warps * (it + 1)))
                            else:
                                p.extend(("wait_count", f"stored{c}.{w}", it + 1) for w in range(epilogue_warps))
                        if g > 0 and "pusher_skips_read_wait" not in mut:
                            p.append(("wait_read", 1))
                        p.append(("expect", f"push{c}.{g % 2}", push_bytes))
                        p.append(("tma_load", c, parts, f"staging{c}.{g % 2}", push_bytes, f"push{c}.{g % 2}"))
                        # (in the kernel the stores of chunk g - 1 are issued before this load; their
                        # order against it is what wait_read establishes, so the program order here is equivalent)
                        if "pusher_skips_load_wait" not in mut:
                            p.append(("wait", f"push{c}.{g % 2}", g // 2 + (1 if "pusher_wrong_parity" in mut else 0)))
                        p.append(("tma_store", c, f"staging{c}.{g % 2}"))
                pushed += push_chunks
            it += 1
    return programs, barriers


def signal_schedule(ctas: int = 4, chunks: int = 3, mutations=()):
    """The end of a several-destination launch with completion counters, and the owner of one
    destination waiting for it (cute_b200_gemm_tn_multi_signal / cute_b200_wait_signal).

    Every CTA's pusher thread stores its chunks into the peer's rows of C (bulk stores from a
    staging buffer it has filled), waits for all its bulk groups, and passes the CTA's closing
    barrier; the CTA's first thread then counts the CTA in on the device's counter; whoever
    brings that counter to the number of CTAs adds 1 to the counter in the peer's memory; the
    peer's waiting kernel polls that counter and then reads the rows.  Mutations:
      "signal_without_store_wait"   the pusher does not wait for its bulk stores before the barrier
      "signal_before_all_ctas"      the remote counter is raised when one CTA is still missing
      "peer_reads_without_waiting"  the owner reads its rows without polling the counter
      "peer_expects_another_sender" the owner waits for one count more than anybody sends
    """
    mut = set(mutations)
    programs, barriers = {}, {}
    for c in range(ctas):
        p = programs[f"pusher{c}"] = []
        for ch in range(chunks):
            p.append(("st", f"staging{c}.{ch}"))                     # stands for the TMA load that fills the buffer
            p.append(("tma_store", c, f"staging{c}.{ch}", f"peer_c.{c}.{ch}"))
        if "signal_without_store_wait" not in mut:
            p.append(("wait_all",))
        p.append(("signal", f"cta_barrier{c}"))                      # the closing __syncthreads of the CTA
        t = programs[f"thread0.{c}"] = []
        t.append(("wait_count", f"cta_barrier{c}", 1))
        t.append(("signal", "device_done"))
    last = programs["last_cta"] = []                                 # the thread that sees the count complete
    last.append(("wait_count", "device_done", ctas - (1 if "signal_before_all_ctas" in mut else 0)))
    last.append(("signal", "peer_counter"))
    owner = programs["owner"] = []
    if "peer_reads_without_waiting" not in mut:
        owner.append(("wait_count", "peer_counter", 2 if "peer_expects_another_sender" in mut else 1))
    for c in range(ctas):
        for ch in range(chunks):
            owner.append(("ld", f"peer_c.{c}.{ch}"))
    return programs, barriers


def check_signal(seeds=range(6), **kw) -> None:
    programs, barriers = signal_schedule(**kw)
    for seed in seeds:
        run(programs, barriers, seed=seed)
        run(programs, barriers, seed=seed, max_burst=2)


def cluster_sum_schedule(kc: int = 2, warps: int = 8, mutations=()):
    """The k split that is summed inside a cluster (GemmParams::kc): each of the kc CTAs holds the partial
    sums of its k range; every epilogue warp writes its part of them to its CTA's shared memory, all
    threads of the cluster meet at a cluster barrier, every warp then reads its rows from every CTA's
    shared memory and stores them to C, and a second cluster barrier in the teardown keeps each CTA's
    shared memory alive until all have read it (the final write below stands for its release).
    Mutations:
      "sum_before_barrier"     a warp reads the other CTAs' partial sums without the first cluster barrier
      "barrier_of_one_cta"     the first barrier counts only the warps of the own CTA
      "exit_without_barrier"   a CTA releases its shared memory without the second cluster barrier
      "a_warp_skips_barrier"   one warp never arrives (what the bounded waits' fall-through prevents): deadlock
    """
    mut = set(mutations)
    programs, barriers = {}, {}
    total = kc * warps
    for c in range(kc):
        for w in range(warps):
            prog = programs[f"epi{c}.{w}"] = []
            prog.append(("st", f"part{c}.{w}"))                                  # TMEM -> this CTA's shared memory
            if not ("a_warp_skips_barrier" in mut and (c, w) == (kc - 1, warps - 1)):
                prog.append(("signal", "exchange"))
            if "sum_before_barrier" not in mut:
                prog.append(("wait_count", "exchange", warps if "barrier_of_one_cta" in mut else total))
            for c2 in range(kc):                                                 # its rows of every CTA's partial sums
                for w2 in range(warps):
                    prog.append(("ld", f"part{c2}.{w2}"))
            prog.append(("st", f"c.{c}.{w}"))
            prog.append(("signal", "teardown"))
            if "exit_without_barrier" not in mut:
                prog.append(("wait_count", "teardown", total))
            prog.append(("st", f"part{c}.{w}"))                                  # the CTA exits: its shared memory is reused
    return programs, barriers


def check_cluster_sum(seeds=range(6), **kw) -> None:
    programs, barriers = cluster_sum_schedule(**kw)
    for seed in seeds:
        run(programs, barriers, seed=seed)
        run(programs, barriers, seed=seed, max_burst=2)


def tiling_from_library(info, cta_group: int) -> dict:
    """gemm_schedule's arguments for a tiling as the compiled kernel has it: `info`
    is the cute_b200_gemm_layout the library reports (ring depth, stage bytes,
    accumulator halves and buffers, epilogue warps, barrier counts, pusher chunk)."""
    assert (info.full_arrivals, info.empty_arrivals, info.tmem_full_arrivals) == (1, 1, 1), \
        "the schedule models one producer arrival, one commit per stage and one per accumulator"
    assert info.stage_bytes == info.k_blocks_per_stage * (info.a_block_bytes + info.b_block_bytes)
    return dict(cta_group=cta_group, stages=info.stages, mh=info.accumulator_halves, acc_bufs=info.accumulator_buffers,
                stage_bytes=info.a_block_bytes + info.b_block_bytes, kps=info.k_blocks_per_stage,
                epilogue_warps=info.epilogue_warps, tmem_empty_arrivals=info.tmem_empty_arrivals,
                expect_tx=info.full_expect_tx_bytes_per_k_block, push_bytes=info.push_chunk_bytes)


def check_gemm(seeds=range(4), **kw) -> None:
    """Run the schedule under several interleavings; raises ProtocolError on the first violation."""
    programs, barriers = gemm_schedule(**kw)
    for seed in seeds:
        run(programs, barriers, seed=seed)
        run(programs, barriers, seed=seed, max_burst=3)
