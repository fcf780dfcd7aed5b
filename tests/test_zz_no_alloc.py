"""The allocation-free token permutation, nvk_b200_moe_permute_static.

Hosts that have no device memory left to allocate (a server whose KV-cache pool took all of it), that
cannot pay for an allocation's device-wide synchronisation inside the decode loop, or whose FFI rule is
that the C side never allocates, call this entry point instead of nv_kernels_moe_permute: it needs no
scratch argument because its counters live in a fixed array inside the library.  The test also
passes on its own in a fresh process (its first call does the one-time address look-up).
"""
import numpy as np
import pytest
import torch

from tests import _util as U

pytestmark = pytest.mark.gpu


def _permute(entry, topk, n_tok, k, E, with_scratch):
    dt = U.dev(topk)
    perm = torch.full((n_tok * k,), -7, dtype=torch.int32, device="cuda")
    offs = torch.full((E + 1,), -7, dtype=torch.int32, device="cuda")
    inv = torch.full((n_tok * k,), -7, dtype=torch.int32, device="cuda")
    args = [U.stream(), dt.data_ptr(), perm.data_ptr(), offs.data_ptr(), inv.data_ptr()]
    keep = None
    if with_scratch:
        keep = torch.zeros(E, dtype=torch.int32, device="cuda")
        args.append(keep.data_ptr())
    rc = U.ffi.call(entry, *args, n_tok, k, E)
    assert rc == 0
    torch.cuda.synchronize()
    return perm.cpu().numpy(), offs.cpu().numpy(), inv.cpu().numpy()


def test_static_permute_matches_the_scratch_version_twice_in_a_row():
    U.require_gpu()
    rng = np.random.default_rng(123)
    # two different problems back to back: the second must not see the first one's counters
    for n_tok, k, E in [(64, 8, 128), (16, 4, 24)]:
        topk = np.stack([rng.permutation(E)[:k] for _ in range(n_tok)]).astype(np.int32)
        want = _permute("nv_kernels_moe_permute", topk, n_tok, k, E, with_scratch=True)
        got = _permute("nvk_b200_moe_permute_static", topk, n_tok, k, E, with_scratch=False)
        for a, b in zip(got, want):
            assert np.array_equal(a, b)  # integer outputs: bit-exact
        # and it is a valid permutation in its own right
        perm, offs, inv = got
        counts = np.bincount(topk.ravel(), minlength=E)
        assert np.array_equal(offs, np.concatenate([[0], np.cumsum(counts)]))
        assert sorted(inv) == list(range(n_tok * k))
        # checked on its own too, not only against the other entry point: the stable sort by expert
        order = np.argsort(topk.ravel(), kind="stable")
        assert np.array_equal(perm, (order // k).astype(np.int32))
        assert np.array_equal(inv[order], np.arange(n_tok * k, dtype=np.int32))


def test_static_permute_refuses_more_experts_than_the_array_holds():
    U.require_gpu()
    t = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = t.data_ptr()
    assert U.ffi.call("nvk_b200_moe_permute_static", U.stream(), p, p, p, p, 4, 2, 4097) == -3
    assert U.ffi.call("nvk_b200_moe_permute_static", U.stream(), p, p, p, p, 0, 2, 8) == 0  # empty: no-op
    torch.cuda.synchronize()
