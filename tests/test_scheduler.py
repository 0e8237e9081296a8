import pytest

from flextrain_b200.scheduler import GreedySnakeBlockScheduler, LLMTask


def pairs(tasks):
    return [(t.unit, t.micro_batch) for t in tasks]


def test_golden_order_3_micro_batches_4_units():
    s = GreedySnakeBlockScheduler(3, 4)
    assert pairs(s.forward_tasks) == [(0, 0), (0, 1), (0, 2), (1, 2), (1, 1), (1, 0), (2, 0), (2, 1), (2, 2)]
    assert pairs(s.backward_tasks) == [(3, 2), (3, 1), (3, 0), (2, 0), (2, 1), (2, 2), (1, 2), (1, 1),
                                       (1, 0), (0, 0), (0, 1), (0, 2)]
    assert all(t.is_forwarding for t in s.forward_tasks)
    assert not any(t.is_forwarding for t in s.backward_tasks)


def test_iteration_protocol_and_properties():
    s = GreedySnakeBlockScheduler(3, 4)
    fwd = list(s)
    assert pairs(fwd) == pairs(s.forward_tasks)
    seen_new_unit = []
    for t in s:                     # backward sweep
        seen_new_unit.append(s.new_unit_entered)
        assert s.curr_task == t
        assert s.in_last_unit == (t.unit == 3)
        assert s.in_first_unit == (t.unit == 0)
    assert seen_new_unit == [True, False, False] * 4
    assert s.next_task == s.tasks[0]          # wraps to the first task of the next step
    assert pairs(list(s)) == pairs(s.forward_tasks)   # next step starts over


@pytest.mark.parametrize("mb,units", [(1, 1), (1, 5), (4, 1), (2, 2), (5, 7)])
def test_every_pair_once_per_pass_and_snake_turns(mb, units):
    s = GreedySnakeBlockScheduler(mb, units)
    assert len(s.forward_tasks) == mb * (units - 1)
    assert len(s.backward_tasks) == mb * units
    assert sorted(pairs(s.forward_tasks)) == [(u, m) for u in range(units - 1) for m in range(mb)]
    assert sorted(pairs(s.backward_tasks)) == [(u, m) for u in range(units) for m in range(mb)]
    tasks = s.tasks
    for a, b in zip(tasks[:-1], tasks[1:]):
        if a.unit != b.unit:                   # the turn keeps the micro-batch
            assert a.micro_batch == b.micro_batch


def test_rejects_empty():
    with pytest.raises(ValueError):
        GreedySnakeBlockScheduler(0, 3)
