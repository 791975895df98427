"""The launcher's rule for programmatic dependent launch, without a GPU (the library loads on a CPU; nothing is launched).

A kernel that overlaps a predecessor with a large shared-memory allocation inherits an SM with little L1, and so
does every kernel that overlaps it in turn; a kernel that wants L1 (the decode product) is launched plainly then.
"""
import pytest

PLAIN, DEPENDENT, WANTS_L1 = 0, 1, 2
SMALL, LARGE = 8 * 1024, 100 * 1024


@pytest.fixture()
def plan():
    from jllm_serve_b200.csrc import ops
    ops.set_dependent_launch(True)
    ops.launch_plan(0, PLAIN)                      # a plain launch: the SMs drain, the record is clean
    yield ops.launch_plan
    ops.launch_plan(0, PLAIN)


def test_products_overlap_one_another(plan):
    assert not plan(SMALL, PLAIN)
    for _ in range(4):
        assert plan(SMALL, WANTS_L1)
        assert plan(SMALL, DEPENDENT)


def test_a_product_behind_a_large_kernel_waits_for_the_sms_to_drain(plan):
    assert plan(LARGE, DEPENDENT)                   # the attention itself may overlap what is before it
    assert not plan(SMALL, WANTS_L1)                # the product behind it may not
    assert plan(SMALL, WANTS_L1)                    # the one after that may again


def test_the_small_kernel_in_between_carries_the_split_along(plan):
    assert plan(LARGE, DEPENDENT)
    assert plan(SMALL, DEPENDENT)                   # the combine does not care about L1 and overlaps the attention
    assert plan(SMALL, DEPENDENT)
    assert not plan(SMALL, WANTS_L1)                # but the SMs have not drained since the large kernel
    assert plan(SMALL, WANTS_L1)


def test_a_plain_launch_in_between_clears_the_record(plan):
    assert plan(LARGE, DEPENDENT)
    assert not plan(SMALL, PLAIN)
    assert plan(SMALL, WANTS_L1)


def test_large_kernels_overlap_one_another(plan):
    assert plan(LARGE, DEPENDENT)
    assert plan(LARGE, DEPENDENT)
    assert not plan(SMALL, WANTS_L1)


def test_nothing_overlaps_when_dependent_launch_is_off(plan):
    from jllm_serve_b200.csrc import ops
    ops.set_dependent_launch(False)
    try:
        assert not plan(SMALL, DEPENDENT)
        assert not plan(LARGE, DEPENDENT)
        assert not plan(SMALL, WANTS_L1)
    finally:
        ops.set_dependent_launch(True)
