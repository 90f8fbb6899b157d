"""Host-side logic of ``Compressgnn_Cluster`` that needs no GPU: the refresh schedule, the
assignment cache and the argument rules (exception classes pinned by the reference's
tests/test_transformation.py:90-107)."""
import pytest
import torch

from compressgnn_b200.layer.cluster import (Assignment, AssignmentCache, AssignmentSignature,
                                             Compressgnn_Cluster, RefreshSchedule)


def test_fixed_schedule_counts_epochs():
    s = RefreshSchedule('fixed', 5, 1, 10, None)
    assert s.needs_epoch and s.interval == 5 and s.epoch is None
    assert s.advance(0) is False
    assert not s.expired(0)
    s.advance(4)
    assert not s.expired(0)
    s.advance(5)
    assert s.expired(0) and not s.expired(5)
    assert s.advance(2) is True      # the clock went backwards: a new run
    assert s.epoch == 2
    assert not RefreshSchedule('fixed', 1, 1, 10, None).needs_epoch


def test_loss_schedule_follows_the_loss():
    s = RefreshSchedule('loss', 1, 1, 10, 0.1)
    assert s.needs_epoch and s.interval == 1
    s.advance(0, loss=1.0)
    assert s.interval == 1           # nothing to compare with yet
    s.advance(1, loss=1.0)
    assert s.interval == 10          # flat loss: keep the assignment as long as allowed
    s.advance(1, loss=5.0)
    assert s.interval == 10          # one update per epoch
    s.advance(2, loss=2.0)
    assert s.interval == 1           # a jump of ten tau
    s.advance(3, loss=2.05)        # exp(-0.5) = 0.607 -> 1 + 9 * 0.607 = 6.46 -> 6
    assert s.interval == 6
    with pytest.raises(TypeError):
        s.advance(4, loss=torch.tensor(1.0))
    with pytest.raises(ValueError):
        s.advance(5, loss=float("nan"))
    with pytest.raises(ValueError):
        s.advance(-1)
    s.restart()
    assert s.epoch is None and s.interval == 1


@pytest.mark.parametrize("kwargs", [
    dict(refresh_policy='sometimes'), dict(refresh_interval=0), dict(q_min=0), dict(q_min=4, q_max=3),
    dict(refresh_policy='loss'), dict(refresh_policy='loss', tau_loss=0.0),
    dict(refresh_policy='loss', tau_loss=float("inf"))])
def test_constructor_rejects_bad_schedules(kwargs):
    with pytest.raises(ValueError):
        Compressgnn_Cluster(7, 4, **kwargs)


def test_constructor_and_input_rules_on_cpu():
    for bits in (-1, 31):
        with pytest.raises(ValueError):
            Compressgnn_Cluster(7, bits)
    c = Compressgnn_Cluster(7, 4, refresh_interval=5)
    assert c.random_vectors.shape == (7, 4) and "random_vectors" in c.state_dict()
    assert (c.refresh_interval, c.refresh_policy, c.q_min, c.q_max, c.current_interval) == (5, 'fixed', 1, 10, 5)
    with pytest.raises(ValueError):      # reuse across epochs without an epoch
        c(torch.zeros(3, 7))
    with pytest.raises(ValueError):      # wrong width
        c(torch.zeros(3, 8), epoch=0)
    with pytest.raises(ValueError):      # wrong dtype
        c(torch.zeros(3, 7, dtype=torch.float64), epoch=0)
    with pytest.raises(RuntimeError):    # CPU tensors: there is no CPU path
        c(torch.zeros(3, 7), epoch=0)
    assert c.set_epoch(3) is c


def test_assignment_cache_matches_on_the_signature():
    cache = AssignmentCache()
    sig = AssignmentSignature((10, 7), torch.float32, "graph-A", 1234, 0)
    a = Assignment(torch.zeros(10, dtype=torch.int64), torch.zeros(2, dtype=torch.int32), 1, sig, 0)
    slot = (True, torch.device("cpu"), 0)
    assert cache.lookup(slot, sig) is None
    cache.keep(slot, a)
    assert cache.lookup(slot, sig) is a
    assert cache.lookup((False,) + slot[1:], sig) is None                       # eval has its own slot
    for other in (AssignmentSignature((11, 7), torch.float32, "graph-A", 1234, 0),
                  AssignmentSignature((10, 7), torch.float64, "graph-A", 1234, 0),
                  AssignmentSignature((10, 7), torch.float32, "graph-B", 1234, 0),
                  AssignmentSignature((10, 7), torch.float32, "graph-A", 1234, 1)):
        assert cache.lookup(slot, other) is None
    cache.clear()
    assert cache.lookup(slot, sig) is None
