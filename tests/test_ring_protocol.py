"""The barrier protocol of the tcgen05 product's shared-memory ring (csrc/gemm_tc.cu), as a model on the host under
random schedules: producers that fill a stage when its last user has freed it, loads that land out of order, MMA
issuers that wait for a stage's fill by the barrier's PARITY (mbarrier.try_wait.parity tells an odd fill from an
even one, not a fill from the one two fills later), an epilogue and two accumulator buffers.

What the model is for: the rule that a stage has ONE consumer.  With one issuer (the kernel as it is) it holds
trivially.  With two issuers that take every other K block it holds only if the parity that assigns a K block to
an issuer is also the parity of its stage: an even number of stages, and blocks counted over all units of the CTA.
Assigning by the block's index within its unit (or an odd number of stages) lets the faster issuer reach a stage
two fills early, which the parity cannot see; that version of the kernel failed on the GPU."""
import random

import pytest


def simulate(stages, blocks_per_unit, units, issuers, assign, seed):
    """True if every schedule step keeps the invariants and all roles finish; else (False, why)."""
    rng = random.Random(seed)
    total = blocks_per_unit * units
    full_phase, empty_phase, landed = [0] * stages, [0] * stages, {}
    acc_full_phase, acc_full_arrivals, acc_empty_phase = [0, 0], [0, 0], [0, 0]
    issued, in_flight = {"W": 0, "X": 0}, []
    issuer = {i: [0, 0, False] for i in range(issuers)}        # unit, block within the unit, waited for the buffer
    drained, done = 0, set()

    def passes(phases_completed, parity):                       # mbarrier.try_wait.parity
        return (phases_completed & 1) != parity

    def takes(who, it, block):
        if issuers == 1:
            return True
        return ((block if assign == "within the unit" else it) & 1) == who

    roles = ["W", "X", "land", "drain"] + [f"issue{i}" for i in range(issuers)]
    for _ in range(300000):
        if len(done) == 3 + issuers and not in_flight:
            return True, None
        role = rng.choice(roles)
        if role in ("W", "X"):
            it = issued[role]
            if it >= total:
                done.add(role)
                continue
            stage = it % stages
            if it >= stages and not passes(empty_phase[stage], ((it // stages) & 1) ^ 1):
                continue
            in_flight.append(it)
            issued[role] = it + 1
        elif role == "land":
            if in_flight:
                it = in_flight.pop(rng.randrange(len(in_flight)))
                landed[it] = landed.get(it, 0) + 1
                if landed[it] == 2:
                    if full_phase[it % stages] != it // stages:
                        return False, f"the fills of stage {it % stages} complete out of turn at block {it}"
                    full_phase[it % stages] += 1
        elif role == "drain":
            if drained >= units:
                done.add(role)
                continue
            buffer, use = drained & 1, drained >> 1
            if passes(acc_full_phase[buffer], use & 1):
                if acc_full_phase[buffer] != use + 1:
                    return False, f"the epilogue reads buffer {buffer} before unit {drained} is complete"
                acc_empty_phase[buffer] += 1
                drained += 1
        else:
            who = int(role[5:])
            unit, block, waited = issuer[who]
            if unit >= units:
                done.add(role)
                continue
            buffer, use = unit & 1, unit >> 1
            if not waited:
                if not passes(acc_empty_phase[buffer], (use & 1) ^ 1):
                    continue
                issuer[who][2] = True
            if block >= blocks_per_unit:
                acc_full_arrivals[buffer] += 1
                if acc_full_arrivals[buffer] == issuers:
                    acc_full_arrivals[buffer] = 0
                    acc_full_phase[buffer] += 1
                issuer[who] = [unit + 1, 0, False]
                continue
            it = unit * blocks_per_unit + block
            if not takes(who, it, block):
                issuer[who][1] = block + 1
                continue
            stage = it % stages
            if not passes(full_phase[stage], (it // stages) & 1):
                continue
            if full_phase[stage] != it // stages + 1:
                return False, f"issuer {who} multiplies stage {stage} for block {it}, which has not landed"
            empty_phase[stage] += 1
            issuer[who][1] = block + 1
    return False, "no progress"


SHAPES = [(blocks, units) for blocks in (1, 2, 3, 9, 32, 64) for units in (1, 2, 3, 4)]


@pytest.mark.parametrize("stages", [2, 3, 5, 8, 12])
def test_one_issuer_sees_every_fill_in_turn(stages):
    for blocks, units in SHAPES:
        for seed in range(4):
            assert simulate(stages, blocks, units, 1, None, seed) == (True, None), (blocks, units, seed)


@pytest.mark.parametrize("stages", [2, 4, 8, 12])
def test_two_issuers_with_one_consumer_per_stage(stages):
    for blocks, units in SHAPES:
        for seed in range(4):
            assert simulate(stages, blocks, units, 2, "over the CTA", seed) == (True, None), (blocks, units, seed)


def test_two_issuers_that_share_a_stage_are_caught_by_the_model():
    """Five stages, one unit of 64 blocks (the product that failed on the GPU), and units of an odd number of
    blocks with an even number of stages: some schedules reach a stage two fills early."""
    early = [simulate(5, 64, 1, 2, "within the unit", seed)[1] for seed in range(40)]
    assert any(why and "has not landed" in why for why in early)
    early = [simulate(2, 3, 2, 2, "within the unit", seed)[1] for seed in range(40)]
    assert any(why and "has not landed" in why for why in early)
