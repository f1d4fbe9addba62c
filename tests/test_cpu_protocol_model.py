"""The signalling protocol of the fused kernels, checked as a host-thread model (same
epoch words, `done` chain and acquire/release structure; see csrc/runtime/protocol_model.cc).
compute-sanitizer is not available on the GPU pool, so this is where ordering mistakes in
the protocol itself would show."""
import pytest

import bagua_core_b200 as bb


@pytest.mark.parametrize("nranks,blocks", [(2, 1), (2, 3), (3, 2), (4, 4), (8, 2)])
def test_random_schedules_never_corrupt_or_hang(nranks, blocks):
    for seed in range(3):
        r = bb._C.protocol_model_check(nranks, blocks, 60, seed=seed)
        assert r == {"errors": 0, "timeouts": 0, "ops": 60}, (nranks, blocks, seed, r)


@pytest.mark.parametrize("nranks,blocks", [(2, 1), (2, 3), (3, 2), (4, 2), (5, 3), (8, 4)])
def test_every_collective_kernel_in_random_order(nranks, blocks):
    """Random sequences over all kernels of the communicator (all-reduces, all-gather, all-to-all,
    reduce-scatter through staging and with direct peer access, both broadcasts, barrier), each
    with the kernels' own index arithmetic: every value that arrives is the expected one."""
    for seed in range(3):
        r = bb._C.protocol_model_check(nranks, blocks, 80, seed=seed, mix=True)
        assert r == {"errors": 0, "timeouts": 0, "ops": 80}, (nranks, blocks, seed, r)


def test_mixed_sequences_need_the_done_chain():
    errors = sum(bb._C.protocol_model_check(4, 2, 200, seed=s, use_done_chain=False, mix=True)["errors"]
                 for s in range(4))
    assert errors > 0


def test_adversarial_delay_is_safe_with_the_done_chain_and_unsafe_without():
    """A rank that lingers in the copy-out of a two-shot op while its peer starts a one-shot op
    over the same staging addresses: the `done` chain is exactly what keeps that safe."""
    safe = bb._C.protocol_model_check(2, 1, 20, seed=1, use_done_chain=True, slow_rank=0)
    assert safe["errors"] == 0 and safe["timeouts"] == 0
    unsafe = bb._C.protocol_model_check(2, 1, 20, seed=1, use_done_chain=False, slow_rank=0)
    assert unsafe["errors"] > 0
