"""The allocation-free Gram entry point against the allocating one.

Some callers cannot allocate device memory when they call the library (they
live inside another framework's memory pool, or run a loop with a fixed memory
budget), so ``dnpeff_op_gram_noalloc`` keeps its partial sums in a fixed array
inside the library.  Two calls in a row share that array; the second must not
be disturbed by what the first left there.  This file is collected last so a
run that stops at the first failure has already run everything else.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_gram_noalloc_matches_gram_twice_in_a_row():
    import torch
    from npeff_ref_b200._lib import lib, check
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    st = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(2024)
    # second call: different shape and a smaller footprint than the first, so
    # stale partials of the first call sit right behind the ones it uses
    for rows, r in [(30000, 128), (4097, 64)]:
        X = torch.from_numpy(rng.random((rows, r), dtype=np.float32)).cuda()
        want = torch.full((r, r), float("nan"), device="cuda")
        got = torch.full((r, r), float("nan"), device="cuda")
        check(lib().dnpeff_op_gram(X.data_ptr(), rows, r, want.data_ptr(), st))
        check(lib().dnpeff_op_gram_noalloc(X.data_ptr(), rows, r, got.data_ptr(), st))
        torch.cuda.synchronize()
        w, g = want.cpu().numpy(), got.cpu().numpy()
        # same tolerance as the Gram parity test: 3e-6 of the largest entry
        assert np.abs(g - w).max() <= 3e-6 * np.abs(w).max()
        ref = X.cpu().numpy().astype(np.float64)
        assert np.abs(g - ref.T @ ref).max() <= 3e-6 * np.abs(w).max()


@pytest.mark.parametrize("rows,r", [(200000, 128), (10000, 1024)])
def test_gram_noalloc_longer_slabs_when_the_default_split_does_not_fit(rows, r):
    """From about 131 000 rows at rank 128, or 8 000 rows at rank 1024, the slab split
    dnpeff_op_gram would use needs more than the fixed 16 MiB: the entry point then
    cuts the rows into fewer, longer slabs.  Same comparison as above, twice in a row."""
    import torch
    from npeff_ref_b200._lib import lib, check
    torch.cuda.set_device(0)
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(rows + r)
    X = torch.rand((rows, r), generator=g, device="cuda")
    ref = (X.double().T @ X.double()).cpu().numpy()
    want = torch.full((r, r), float("nan"), device="cuda")
    check(lib().dnpeff_op_gram(X.data_ptr(), rows, r, want.data_ptr(), st))
    for _ in range(2):
        got = torch.full((r, r), float("nan"), device="cuda")
        check(lib().dnpeff_op_gram_noalloc(X.data_ptr(), rows, r, got.data_ptr(), st))
        torch.cuda.synchronize()
        gnp = got.cpu().numpy()
        assert np.abs(gnp - want.cpu().numpy()).max() <= 3e-6 * np.abs(ref).max()
        assert np.abs(gnp - ref).max() <= 3e-6 * np.abs(ref).max()
        assert np.array_equal(gnp, gnp.T)


def test_gram_noalloc_rejects_rank_beyond_limit():
    import torch
    from npeff_ref_b200._lib import lib
    torch.cuda.set_device(0)
    X = torch.zeros((4, 1028), device="cuda")
    G = torch.zeros((1028, 1028), device="cuda")
    code = lib().dnpeff_op_gram_noalloc(X.data_ptr(), 4, 1028, G.data_ptr(), None)
    assert code == -5
    assert b"limit" in lib().dnpeff_last_error()
