"""The barrier protocols of the tcgen05 kernels, restated as little programs and explored over EVERY interleaving,
without a GPU.  First and in most detail the prefill attention kernel (hymt2sharp_b200/csrc/attention_prefill_tc.cu);
the decode attention and the persistent matrix product follow at the end.

Why: a wait on an mbarrier names a parity, and a parity cannot tell a phase from the one two later.  A reader that
falls two phases behind its barrier waits for ever; one that is a phase early passes at once.  Whether that can
happen does not depend on likelihoods (a thread may be kept from running for any length of time) but on who has to
wait for whom, and that can be enumerated.  The roles, as in the kernel:

  producer       Q with K(0); then for every tile i: wait "stage i mod 2 free" (tile i - 2), copy K(i + 1) with V(i)
  score issuer   S(0); then for i: wait copy i, release its hold on the stage, wait P·V(i - 2), wait P(i - 1), issue S(i + 1)
  P·V issuer     for i: wait P(i), wait copy i, issue P·V(i), whose completion frees the stage and completes O's barrier
  softmax        for i: wait S(i), sometimes wait P·V(i - 1) (a maximum rose), on the last tile sometimes wait copy i,
                 announce P(i); at the end wait P·V of the last tile

Copies land and products complete at any later time (products of one issuer in order).  A first version with two
barriers for P, two for O and the stage held by P·V alone met the never-ending wait on the device; the exploration
finds it in that version within milliseconds, and finds none in the kernel's.

The numbers that the little programs are built from (stages, K slots, barriers per purpose, holders of a stage,
accumulators, issuers) are not written here: they come out of the compiled kernels (ops.protocol_numbers, which
returns the .cu files' own constants), so a change of one of them in a kernel changes what is explored."""
import pytest

from hymt2sharp_b200.kernels import ops

NUMBERS = ops.protocol_numbers()


def explore(roles, sizes, arrivals_needed=None):
    """roles: programs of ("wait" | "wait or not", barrier, index, phase), ("arrive", barrier, index),
    ("copy", barrier, index) — lands at any later time — and ("issue", queue, [(barrier, index), ...]) — completes at
    any later time after the products issued before it on the same queue, and then arrives at its barriers.
    sizes: barriers of each name; arrivals_needed: arrivals that complete a phase (1 unless named).
    Returns None when no interleaving goes wrong, else a sentence about the first one found that does."""
    arrivals_needed = arrivals_needed or {}
    at, total = {}, 0
    for name, n in sizes.items():
        at[name] = total
        total += n
    queues = sorted({op[1] for role in roles for op in role if op[0] == "issue"})

    def arrive(done, held, bar, idx):
        done, held = list(done), list(held)
        held[at[bar] + idx] += 1
        if held[at[bar] + idx] == arrivals_needed.get(bar, 1):
            held[at[bar] + idx] = 0
            done[at[bar] + idx] += 1
        return tuple(done), tuple(held)

    # (each role's place, completed phases of every barrier, arrivals at the open phases, copies in flight, products in flight)
    first = ((0,) * len(roles), (0,) * total, (0,) * total, (), tuple(() for _ in queues))
    seen, todo = {first}, [first]
    while todo:
        places, done, held, copies, issued = todo.pop()
        after = []
        for r, role in enumerate(roles):
            if places[r] >= len(role):
                continue
            op = role[places[r]]
            moved = places[:r] + (places[r] + 1,) + places[r + 1:]
            if op[0] in ("wait", "wait or not"):
                _, bar, idx, phase = op
                complete = done[at[bar] + idx]
                if op[0] == "wait or not":
                    after.append((moved, done, held, copies, issued))
                if (complete & 1) != (phase & 1):      # what the parity test sees
                    if complete != phase + 1:
                        return f"role {r} passes its wait for phase {phase} of {bar}[{idx}] with {complete} phases complete"
                    after.append((moved, done, held, copies, issued))
            elif op[0] == "arrive":
                d, h = arrive(done, held, op[1], op[2])
                after.append((moved, d, h, copies, issued))
            elif op[0] == "copy":
                after.append((moved, done, held, tuple(sorted(copies + ((op[1], op[2]),))), issued))
            else:
                q = queues.index(op[1])
                after.append((moved, done, held, copies, issued[:q] + (issued[q] + (tuple(op[2]),),) + issued[q + 1:]))
        for j, (bar, idx) in enumerate(copies):            # a copy lands
            d, h = arrive(done, held, bar, idx)
            after.append((places, d, h, copies[:j] + copies[j + 1:], issued))
        for q in range(len(queues)):                       # the oldest product of a queue is complete
            if issued[q]:
                d, h = done, held
                for bar, idx in issued[q][0]:
                    d, h = arrive(d, h, bar, idx)
                after.append((places, d, h, copies, issued[:q] + (issued[q][1:],) + issued[q + 1:]))
        if not after and any(places[r] < len(role) for r, role in enumerate(roles)):
            stuck = [role[places[r]] for r, role in enumerate(roles) if places[r] < len(role)]
            return f"nothing can move any more: {stuck}"
        for state in after:
            if state not in seen:
                seen.add(state)
                todo.append(state)
    return None


def prefill(tiles, p_bars, o_bars, stage_holders, kv_stages=None):
    kv = kv_stages or NUMBERS["prefill"]["kv_stages"]
    assert NUMBERS["prefill"]["s_buffers"] == 2     # the score buffers go by a tile's parity, here as in the kernel
    producer = [("copy", "q", 0)]
    for i in range(tiles):
        if i >= kv:
            producer.append(("wait", "stage_free", i % kv, i // kv - 1))
        producer.append(("copy", "copied", i % kv))
    scores = [("wait", "q", 0, 0), ("issue", "S", [("s_done", 0)])]
    for i in range(tiles - 1):
        scores.append(("wait", "copied", i % kv, i // kv))
        if stage_holders == 2:
            scores.append(("arrive", "stage_free", i % kv))
        if i >= 2:
            scores.append(("wait", "o_done", (i - 2) % o_bars, (i - 2) // o_bars))
        if i >= 1:
            scores.append(("wait", "p_written", (i - 1) % p_bars, (i - 1) // p_bars))
        scores.append(("issue", "S", [("s_done", (i + 1) & 1)]))
    weighted = []
    for i in range(tiles):
        weighted.append(("wait", "p_written", i % p_bars, i // p_bars))
        weighted.append(("wait", "copied", i % kv, i // kv))
        weighted.append(("issue", "PV", [("stage_free", i % kv), ("o_done", i % o_bars)]))
    softmax = []
    for i in range(tiles):
        softmax.append(("wait", "s_done", i & 1, i >> 1))
        if i > 0:
            softmax.append(("wait or not", "o_done", (i - 1) % o_bars, (i - 1) // o_bars))
        if i == tiles - 1:
            softmax.append(("wait or not", "copied", i % kv, i // kv))
        softmax.append(("arrive", "p_written", i % p_bars))
    softmax.append(("wait", "o_done", (tiles - 1) % o_bars, (tiles - 1) // o_bars))
    sizes = {"q": 1, "copied": kv, "stage_free": kv, "s_done": 2, "o_done": o_bars, "p_written": p_bars}
    return explore((producer, scores, weighted, softmax), sizes, {"stage_free": stage_holders})


@pytest.mark.parametrize("tiles", [1, 2, 3, 4, 5, 8, 13, 32])
def test_no_interleaving_of_the_kernels_protocol_goes_wrong(tiles):
    n = NUMBERS["prefill"]     # as compiled: 2 stages, 3 barriers for P (one per K slot), 3 for O, 2 holders of a stage
    assert n["p_bars"] == n["k_slots"]
    assert prefill(tiles, p_bars=n["p_bars"], o_bars=n["o_bars"], stage_holders=n["stage_holders"]) is None


@pytest.mark.parametrize("p_bars, o_bars, stage_holders", [(2, 2, 1), (2, 3, 2), (3, 2, 2), (3, 3, 1)])
def test_each_of_the_three_measures_is_needed(p_bars, o_bars, stage_holders):
    """Two barriers for P (the version that hung on the device), two for O, or a stage that only P·V holds: each
    has an interleaving in which a reader is two phases behind and nothing can move any more."""
    found = [prefill(tiles, p_bars, o_bars, stage_holders) for tiles in (3, 4, 5, 6)]
    assert any(found), found


# ---- the decode attention kernel (hymt2sharp_b200/csrc/attention_decode_tc.cu), one round of a CTA's items ----
#   producer       the first three items' copies at once; then for item n: wait "stage n mod 3 free" (item n - 3), copy K with Q, copy V
#   score issuer   for n: wait K and Q of n, wait "accumulators n mod 2 free" (item n - 2), issue S(n)
#   P·V issuer     for n: wait P(n), wait V(n), issue P·V(n), whose completion completes O's barrier and frees the stage;
#                  at the end it waits for the last stages to be free
#   softmax groups group g takes the items n = g, g + 2, ...: wait S(n), sometimes wait V(n) (rows to clear), announce P(n),
#                  wait O(n), free the accumulators
def decode(items):
    stages = NUMBERS["decode"]["stages"]
    assert NUMBERS["decode"]["accumulators"] == 2   # two groups of softmax warps take turns, here as in the kernel
    producer, scores, weighted, groups = [], [], [], ([], [])
    for n in range(items):
        s, t = n % stages, n & 1
        if n >= stages:
            producer.append(("wait", "stage_free", s, n // stages - 1))
        producer += [("copy", "kq_full", s), ("copy", "v_full", s)]
        scores.append(("wait", "kq_full", s, n // stages))
        if n >= 2:
            scores.append(("wait", "tmem_free", t, (n >> 1) - 1))
        scores.append(("issue", "S", [("s_done", t)]))
        weighted += [("wait", "p_ready", t, n >> 1), ("wait", "v_full", s, n // stages),
                     ("issue", "PV", [("o_done", t), ("stage_free", s)])]
        groups[t].extend([("wait", "s_done", t, n >> 1), ("wait or not", "v_full", s, n // stages), ("arrive", "p_ready", t),
                          ("wait", "o_done", t, n >> 1), ("arrive", "tmem_free", t)])
    for m in range(max(0, items - stages), items):
        weighted.append(("wait", "stage_free", m % stages, m // stages))
    sizes = {"kq_full": stages, "v_full": stages, "stage_free": stages, "s_done": 2, "p_ready": 2, "o_done": 2, "tmem_free": 2}
    return explore((producer, scores, weighted, groups[0], groups[1]), sizes)


@pytest.mark.parametrize("items", [1, 2, 3, 4, 7, 12])
def test_no_interleaving_of_the_decode_attentions_protocol_goes_wrong(items):
    assert decode(items) is None


# ---- the persistent matrix product (hymt2sharp_b200/csrc/gemm_tc.cu): a ring of stages across tiles, two accumulators ----
#   producer   for every k block: wait "stage free" (the block a ring earlier), copy the stage
#   issuer     for every tile j: wait "accumulator j mod 2 drained" (tile j - 2); for its k blocks: wait the stage, issue the
#              MMAs (their completion frees the stage); then the tile's completion fills the accumulator's barrier
#   epilogue   group g, for the tiles g, g + groups, ...: wait the accumulator, drain it, announce it empty; then help with
#              the last tile if it is the other group's
# (the looks ahead at the next stage's barrier are reads of the same reader in the same order: nothing new for this model)
def persistent_gemm(tiles, k_blocks, stages, groups=None):
    groups = groups or NUMBERS["gemm"]["epilogue_groups"]
    producer, issuer, epilogues = [], [], [[] for _ in range(groups)]
    block = 0
    for j in range(tiles):
        if j >= 2:
            issuer.append(("wait", "acc_empty", j & 1, (j >> 1) - 1))
        for _ in range(k_blocks):
            s, use = block % stages, block // stages
            if use > 0:
                producer.append(("wait", "empty", s, use - 1))
            producer.append(("copy", "full", s))
            issuer += [("wait", "full", s, use), ("issue", "MMA", [("empty", s)])]
            block += 1
        issuer.append(("issue", "MMA", [("acc_full", j & 1)]))
        epilogues[j % groups] += [("wait", "acc_full", j & 1, j >> 1), ("arrive", "acc_empty", j & 1)]
    if groups == 2:
        # the CTA's last tile is drained by both groups: the group that does not own it waits for its accumulator too,
        # on a barrier whose earlier phases it has not followed, once it is through with its own tiles
        last = tiles - 1
        epilogues[1 - last % 2].append(("wait", "acc_full", last & 1, last >> 1))
    return explore((producer, issuer, *epilogues), {"full": stages, "empty": stages, "acc_full": 2, "acc_empty": 2})


@pytest.mark.parametrize("tiles, k_blocks, stages", [(1, 1, 4), (3, 2, 4), (5, 3, 2), (6, 4, 5), (4, 9, 4),
                                                     (3, 10, NUMBERS["gemm"]["max_stages"])])
def test_no_interleaving_of_the_persistent_products_protocol_goes_wrong(tiles, k_blocks, stages):
    assert NUMBERS["gemm"]["accumulators"] == 2 and 2 <= stages <= NUMBERS["gemm"]["max_stages"]
    assert NUMBERS["gemm"]["epilogue_groups"] in (1, 2)   # a group per accumulator, or one group for both
    assert persistent_gemm(tiles, k_blocks, stages) is None
    assert persistent_gemm(tiles, k_blocks, stages, groups=1) is None


# ---- the tile kernel of the matrix product with several MMA issuers (few tokens): who may read which stage's barrier ----
#   producer   for every k block i: wait "stage i mod stages free" (block i - stages), copy the stage
#   issuer j   takes some of the k blocks: wait the stage, issue its MMAs into an accumulator of its own (they free the stage)
# "own": issuer j takes the blocks that land in the stages j, j + issuers, ... (what the kernel does); otherwise the blocks
# j, j + issuers, ... round-robin, which was the first version: an issuer then met a stage's barrier only every few phases.
def tile_gemm(blocks, stages, issuers, own):
    producer = []
    takers = [[] for _ in range(issuers)]
    for i in range(blocks):
        s = i % stages
        if i >= stages:
            producer.append(("wait", "empty", s, i // stages - 1))
        producer.append(("copy", "full", s))
        j = s % issuers if own else i % issuers
        takers[j] += [("wait", "full", s, i // stages), ("issue", f"MMA{j}", [("empty", s)])]
    return explore((producer, *takers), {"full": stages, "empty": stages})


@pytest.mark.parametrize("blocks, stages", [(32, 5), (12, 6), (20, 3), (7, 2), (18, 4), (40, NUMBERS["gemm"]["max_stages"])])
@pytest.mark.parametrize("issuers", sorted({1, NUMBERS["gemm"]["issuers"]}))
def test_issuers_that_own_their_stages_never_misread_a_barrier(blocks, stages, issuers):
    assert NUMBERS["gemm"]["issuers_own_stages"] == 1
    assert tile_gemm(blocks, stages, issuers, own=True) is None


def test_three_issuers_taking_turns_over_five_stages_did():
    """The version that ended two launches with a fault: an issuer took a stage whose copy had not landed."""
    assert "passes its wait" in tile_gemm(32, 5, 3, own=False)
