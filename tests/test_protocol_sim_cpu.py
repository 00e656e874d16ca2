"""Synchronisation protocols of the peer-memory kernels emulated with one host thread per rank
(csrc/runtime/protocol_sim.cpp): the shipped parameters are race free under thread jitter, the weaker ones are not."""
import pytest

from rustorch_b200 import _native


@pytest.mark.parametrize("world", [2, 4, 8])
def test_lamport_allreduce_three_slots(world):
    h = _native.host()
    r = h.sim_lamport_allreduce(world, 3000, 48, slots=3, slow_rank=world - 1, slow_us=5, seed=world)
    assert r["checked"] == 3000 * world * 48 and r["mismatches"] == 0 and r["timeouts"] == 0, r


def _exposed(run) -> bool:
    """The broken variants depend on an unlucky interleaving: try several seeds and delays before giving up."""
    for seed in range(8):
        r = run(seed, 10 * (seed + 1))
        if r["mismatches"] + r["timeouts"] > 0:
            return True
    return False


def test_lamport_allreduce_two_slots_race_is_detected():
    h = _native.host()
    if not _exposed(lambda seed, us: h.sim_lamport_allreduce(4, 3000, 48, slots=2, slow_rank=0, slow_us=us, seed=seed)):
        pytest.skip("no thread interleaving on this host exposed the two-slot race")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_reduce_scatter_counters_two_parities(world):
    h = _native.host()
    r = h.sim_epoch_counters(world, 800, blocks=4, tiles=8, parities=2, slow_rank=0, slow_us=5, seed=world)
    assert r["mismatches"] == 0 and r["timeouts"] == 0 and r["checked"] == 800 * world * (world - 1) * 32, r


def test_single_staging_buffer_race_is_detected():
    h = _native.host()
    if not _exposed(lambda seed, us: h.sim_epoch_counters(4, 400, parities=1, slow_rank=0, slow_us=us, seed=seed)):
        pytest.skip("no thread interleaving on this host exposed the single-buffer race")
