"""GPU: the batch loader (origindl_b200/loader.py) and its row-gather kernel (odl_gather_rows) against numpy indexing --
pure data movement, so every comparison is bit-exact.  Batch order, the short last batch and the error on next() past
the end follow DataLoader (src/data/dataloader.cpp:17-146; tests/unit_test/data/test_dataloader.cpp)."""
import numpy as np
import pytest
import torch

import _libs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from origindl_b200 import capi

    capi.init(0)
    yield capi
    capi.device_status()


def dataset(n, features, seed=0):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((n, features)).astype(np.float32), rng.integers(0, 10, n).astype(np.int32)


@pytest.mark.parametrize("n_src,cols,n_idx", [(1000, 784, 256), (37, 13, 100), (5, 4, 1), (300, 8192, 64)])
def test_gather_rows_is_a_row_copy(capi, n_src, cols, n_idx):
    x, t = dataset(n_src, cols, seed=n_src)
    idx = np.random.default_rng(1).integers(0, n_src, n_idx)
    dx, dt, di = torch.from_numpy(x).cuda(), torch.from_numpy(t.astype(np.int64)).cuda(), torch.from_numpy(idx).cuda()
    out, lab = torch.empty(n_idx, cols, device="cuda"), torch.empty(n_idx, dtype=torch.int64, device="cuda")
    capi.call("odl_gather_rows", dx.data_ptr(), cols, n_src, di.data_ptr(), n_idx, cols, out.data_ptr(), cols,
              dt.data_ptr(), lab.data_ptr(), capi.stream_handle())
    capi.device_status()
    assert np.array_equal(out.cpu().numpy(), x[idx]) and np.array_equal(lab.cpu().numpy(), t[idx])


def test_gather_rows_rejects_bad_arguments_and_flags_bad_indices(capi):
    x, t = dataset(16, 8)
    dx, dt = torch.from_numpy(x).cuda(), torch.from_numpy(t.astype(np.int64)).cuda()
    idx = torch.tensor([0, 99, 3, -1], dtype=torch.int64, device="cuda")
    out, lab = torch.full((4, 8), 7.0, device="cuda"), torch.empty(4, dtype=torch.int64, device="cuda")
    with pytest.raises(capi.OdlError):
        capi.call("odl_gather_rows", dx.data_ptr(), 4, 16, idx.data_ptr(), 4, 8, out.data_ptr(), 8, None, None,
                  capi.stream_handle())  # pitch smaller than the row
    with pytest.raises(capi.OdlError):
        capi.call("odl_gather_rows", dx.data_ptr(), 8, 16, idx.data_ptr(), 4, 8, out.data_ptr(), 8, None, lab.data_ptr(),
                  capi.stream_handle())  # labels wanted, none given
    capi.call("odl_gather_rows", dx.data_ptr(), 8, 16, idx.data_ptr(), 4, 8, out.data_ptr(), 8, dt.data_ptr(),
              lab.data_ptr(), capi.stream_handle())
    with pytest.raises(capi.OdlError, match="index out of range"):
        capi.device_status()
    got = out.cpu().numpy()
    assert np.array_equal(got[0], x[0]) and np.array_equal(got[2], x[3]) and not got[1].any() and not got[3].any()
    assert lab.cpu().tolist() == [int(t[0]), -1, int(t[3]), -1]


@pytest.mark.parametrize("resident", [True, False])
def test_sequential_epoch_matches_the_reference_order(capi, resident):
    from origindl_b200.loader import DataLoader

    x, t = dataset(70, 24)
    ld = DataLoader(x.reshape(70, 2, 3, 4), t, 32, shuffle=False, resident=resident)  # samples are flattened
    assert len(ld) == 3
    for epoch in range(2):
        seen = 0
        for want in (32, 32, 6):  # the last batch of an epoch is short
            assert ld.has_next()
            bx, bt = ld.next()
            assert bx.shape == (want, 24) and bt.dtype == torch.int64
            assert np.array_equal(bx.cpu().numpy(), x[seen:seen + want]) and np.array_equal(bt.cpu().numpy(), t[seen:seen + want])
            seen += want
        assert not ld.has_next()
        with pytest.raises(RuntimeError, match="no more data available"):
            ld.next()
        ld.reset()
    ld2 = DataLoader(x, t, 32, shuffle=False, drop_last=True, resident=resident)
    assert len(ld2) == 2 and sum(b[0].shape[0] for b in ld2) == 64
    for l in (ld, ld2):
        l.close()


@pytest.mark.parametrize("resident", [True, False])
def test_shuffled_epochs_are_permutations_and_reproducible(capi, resident):
    from origindl_b200.loader import DataLoader

    x, t = dataset(200, 16)
    x[:, 0] = np.arange(200)  # the first feature names the sample
    a = DataLoader(x, t, 64, shuffle=True, seed=5, resident=resident)
    b = DataLoader(x, t, 64, shuffle=True, seed=5, resident=not resident)
    orders = []
    for epoch in range(2):
        ids = []
        while a.has_next():
            (ax, at), (bx, bt) = a.next(), b.next()
            assert torch.equal(ax, bx) and torch.equal(at, bt)  # both modes deliver the same batches for one seed
            rows = ax[:, 0].cpu().numpy().astype(np.int64)
            assert np.array_equal(ax.cpu().numpy(), x[rows]) and np.array_equal(at.cpu().numpy(), t[rows])
            ids.append(rows)
        ids = np.concatenate(ids)
        assert np.array_equal(np.sort(ids), np.arange(200)) and not np.array_equal(ids, np.arange(200))
        orders.append(ids)
        a.reset(), b.reset()
    assert not np.array_equal(orders[0], orders[1])  # reset() reshuffles (dataloader.cpp:17-36)
    a.close(), b.close()


@pytest.mark.parametrize("resident", [True, False])
def test_reset_in_the_middle_of_an_epoch_starts_a_full_new_epoch(capi, resident):
    from origindl_b200.loader import DataLoader

    x, t = dataset(150, 8)
    x[:, 0] = np.arange(150)
    ld = DataLoader(x, t, 40, shuffle=True, seed=9, resident=resident)
    first = ld.next()[0][:, 0].cpu().numpy().copy()
    ld.reset()  # abandons the 110 samples not yet delivered
    ids = np.concatenate([bx[:, 0].cpu().numpy() for bx, _ in ld]).astype(np.int64)
    assert ids.size == 150 and np.array_equal(np.sort(ids), np.arange(150))
    assert not np.array_equal(ids[:40], first)
    ld.close()


@pytest.mark.parametrize("resident", [True, False])
def test_training_from_the_loader_equals_direct_feeding(capi, resident):
    from origindl_b200.loader import DataLoader
    from origindl_b200.trainer import MLPTrainer

    sizes, batch = [32, 48, 10], 64
    x, t = dataset(64 * 5, 32, seed=2)
    params = _libs.mlp_params(np.random.default_rng(1), sizes)
    direct = MLPTrainer(sizes, batch, optimizer="sgd", lr=0.05, momentum=0.9)
    direct.set_params(params)
    xd, td = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()
    want = [direct.train_step(xd[i * batch:(i + 1) * batch], td[i * batch:(i + 1) * batch]).item() for i in range(5)]
    fed = MLPTrainer(sizes, batch, optimizer="sgd", lr=0.05, momentum=0.9)
    fed.set_params(params)
    ld = DataLoader(x, t, batch, shuffle=False, resident=resident)
    got = []
    while ld.has_next():
        bx, bt = ld.next()
        got.append(fed.train_step(bx, bt).item())
        ld.release()
    assert got == want
    ld.close(), direct.close(), fed.close()


@pytest.mark.parametrize("resident", [True, False])
@pytest.mark.parametrize("shuffle", [True, False])
def test_sharded_loaders_partition_every_epoch(capi, resident, shuffle):
    """shard=(rank, world): the ranks' loaders (same seed) deliver disjoint samples that together cover the epoch, with
    equally many batches per rank."""
    from origindl_b200.loader import DataLoader

    x, t = dataset(210, 8)
    x[:, 0] = np.arange(210)
    world = 4
    loaders = [DataLoader(x, t, 16, shuffle=shuffle, seed=21, resident=resident, shard=(r, world)) for r in range(world)]
    assert len({len(ld) for ld in loaders}) == 1
    for epoch in range(2):
        seen = []
        for ld in loaders:
            ids = np.concatenate([bx[:, 0].cpu().numpy() for bx, _ in ld]).astype(np.int64)
            assert ids.size == 208 // world
            seen.append(ids)
        allids = np.concatenate(seen)
        assert np.unique(allids).size == 208 and allids.max() < 210
    if shuffle:
        with pytest.raises(ValueError, match="explicit seed"):
            DataLoader(x, t, 16, shuffle=True, shard=(0, 2))
    for ld in loaders:
        ld.close()
