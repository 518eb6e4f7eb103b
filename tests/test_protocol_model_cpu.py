"""Exhaustive interleaving check of the cross-GPU flag protocol of the fused ZeRO-2 step (host-side model)."""
import pytest

from rwkvtune_b200.parallel.protocol_model import ProtocolViolation, explore, zero2_step_programs


@pytest.mark.parametrize("world,buckets", [(2, 2), (2, 3), (3, 2)])
def test_bucket_flags_and_barriers_order_every_read(world, buckets):
    programs, words = zero2_step_programs(world, buckets, owner_of_bucket=lambda b: b % world, micro_batches=2)
    states = explore(programs, words)
    assert states > 100          # the exploration really branched


def test_model_catches_a_flag_raised_before_the_data_is_written():
    programs, words = zero2_step_programs(2, 2, owner_of_bucket=lambda b: b % 2, signal_before_write=True)
    with pytest.raises(ProtocolViolation, match="expected version"):
        explore(programs, words)


def test_model_catches_a_missing_barrier_between_micro_batches():
    programs, words = zero2_step_programs(2, 2, owner_of_bucket=lambda b: b % 2, skip_micro_barrier=True)
    with pytest.raises(ProtocolViolation):
        explore(programs, words)


def test_model_reports_deadlock():
    programs = [{"compute": [("wait", 0, 1)]}, {"compute": [("wait", 0, 1)]}]
    with pytest.raises(ProtocolViolation, match="deadlock"):
        explore(programs, 1)
