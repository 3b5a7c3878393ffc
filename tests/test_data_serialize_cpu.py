"""Data pipeline (assertions of ferrum-data's unit tests: dataset.rs:202-269, dataloader.rs:192-264,
sampler.rs:360-458, transform.rs:168-202) and the FERRUM01 container (golden bytes assembled by hand from the
layout of ferrum-serialize/src/{format,io}.rs; the reference has no serializer test)."""
import struct

import numpy as np
import pytest
import torch

import ferrum_b200 as fb
from ferrum_b200 import DType, Tensor, data


class Squares(data.Dataset):
    def __init__(self, n):
        self.n = n

    def len(self):
        return self.n

    def get(self, i):
        return Tensor.from_slice([float(i)]), Tensor.from_slice([float(i * i)])


def test_tensor_dataset_variants():
    ds = data.TensorDataset([Tensor.ones([2])] * 3, [Tensor.zeros([1])] * 3)
    assert ds.len() == 3 and not ds.is_empty() and ds.get(1)[0].shape == (2,)
    with pytest.raises(ValueError):
        data.TensorDataset([Tensor.ones([2])], [])
    st = data.TensorDataset.from_tensors(Tensor.arange(12).reshape([6, 2]), Tensor.arange(6))
    assert st.len() == 6 and st.get(2)[0].to_vec() == [4, 5] and st[5][1].item() == 5
    xb, yb = st.get_batch([0, 3])
    assert xb.to_vec() == [0, 1, 6, 7] and yb.to_vec() == [0, 3]


def test_map_concat_subset_split():
    ds = Squares(10)
    m = data.MapDataset(ds, lambda s: (s[0].mul_scalar(2), s[1]))
    assert m.len() == 10 and m.get(3)[0].item() == 6
    c = data.ConcatDataset([Squares(3), Squares(4)])
    assert c.len() == 7 and c.get(2)[0].item() == 2 and c.get(3)[0].item() == 0 and c.get(6)[0].item() == 3
    s = data.Subset(ds, [9, 1])
    assert s.len() == 2 and s.get(0)[0].item() == 9
    tr, te = data.train_test_split(ds, 0.25, shuffle=False)
    assert tr.len() == 7 and te.len() == 3  # ceil(10 * 0.25)
    tr2, te2 = data.train_test_split(ds, 0.2, shuffle=True, seed=1)
    got = sorted(tr2.indices + te2.indices)
    assert got == list(range(10)) and tr2.len() == 8


def test_dataloader_batches_drop_last_shuffle():
    ds = Squares(10)
    dl = data.DataLoader.new(ds).batch_size(3)
    assert dl.len() == 4 and not dl.is_empty() and dl.dataset() is ds
    batches = list(dl)
    assert [b[0].shape[0] for b in batches] == [3, 3, 3, 1]
    assert batches[0][0].to_vec() == [0, 1, 2]
    dl = data.DataLoader(ds, batch_size=3, drop_last=True)
    assert dl.len() == 3 and len(list(dl.iter())) == 3
    a = [x.to_vec() for x, _ in data.DataLoader(ds, batch_size=10, shuffle=True, seed=7)]
    b = [x.to_vec() for x, _ in data.DataLoader(ds, batch_size=10, shuffle=True, seed=7)]
    assert a == b and a[0] != list(map(float, range(10))) and sorted(a[0]) == list(map(float, range(10)))
    raw = list(data.DataLoader(ds, batch_size=4).collate(None))
    assert isinstance(raw[0], list) and len(raw[0]) == 4 and isinstance(raw[0][0], tuple)  # Vec<Sample>
    par = list(data.DataLoader(ds, batch_size=5, num_workers=2))
    assert par[1][1].to_vec() == [25, 36, 49, 64, 81]
    col = data.CollatedDataLoader.new(data.DataLoader(ds, batch_size=5), lambda ss: len(ss))
    assert list(col) == [5, 5]


@pytest.mark.parametrize("width", [1024, 68, 65, 130])
def test_dataloader_native_rows_of_every_width_arrive_intact(width):
    """Rows of 256 bytes and more leave the worker threads with non-temporal stores in 64-byte pieces (plus an
    ordinary tail); narrower rows and rows that start off a 16-byte boundary take the plain copy.  4096, 272, 260 and
    520 bytes per row cover the four cases."""
    x = torch.arange(300 * width, dtype=torch.float32).view(300, width)
    ds = data.TensorDataset.from_tensors(x, torch.arange(300))
    loader = data.DataLoader(ds).batch_size(32).shuffle(True).seed(3).num_workers(4)
    seen = 0
    for a, b in loader:
        assert torch.equal(a._t, x[b._t])
        seen += b._t.numel()
    assert seen == 300
    loader.close()


def test_dataloader_native_worker_path_matches_the_plain_path():
    """Stacked host tensors + ``num_workers > 0``: rows are gathered by the host library's worker threads into a
    ring of staging slots.  Same batches as the single-threaded path for the same seed, ragged last batch,
    ``repeat`` across epochs, an abandoned iteration, and a sampler that hands out a bad index."""
    import numpy as np

    from ferrum_b200.data import Sampler

    x = torch.arange(1003 * 5, dtype=torch.float32).view(1003, 5)
    y = torch.arange(1003) * 3
    ds = data.TensorDataset.from_tensors(x, y)
    plain = [(a._t.clone(), b._t.clone()) for a, b in data.DataLoader(ds).batch_size(64).shuffle(True).seed(5)]
    native = data.DataLoader(ds).batch_size(64).shuffle(True).seed(5).num_workers(3)
    got = [(a._t, b._t) for a, b in native]
    assert len(got) == len(plain) == 16 and got[-1][0].shape[0] == 1003 - 15 * 64
    for (a, b), (c, d) in zip(got, plain):
        assert torch.equal(a, c) and torch.equal(b, d)
    assert all(torch.equal(a[:, 0] / 5 * 3, b.float()) for a, b in got)
    # second epoch of the same loader reshuffles; repeat never stops and keeps rows intact
    again = torch.cat([b._t for _, b in native])
    assert sorted(again.tolist()) == (torch.arange(1003) * 3).tolist() and not torch.equal(again, torch.cat(
        [b for _, b in got]))
    native.repeat(True).drop_last(True)
    it = iter(native)
    rows = 0
    for _ in range(50):
        a, b = next(it)
        assert a._t.shape == (64, 5) and torch.equal(a._t[:, 0] / 5 * 3, b._t.float())
        rows += 64
    del it                      # abandoned with slots in flight
    assert rows == 3200
    native.repeat(False)
    assert sum(b._t.numel() for _, b in native) == 15 * 64
    it = iter(native)
    next(it)
    native.close()              # closed under a live iterator: the iterator must not touch the freed workers
    del it

    class Bad(Sampler):
        def __init__(self):
            super().__init__(np.array([0, 1, 5000, 2], dtype=np.int64))

    bad = data.DataLoader(ds).batch_size(2).sampler(Bad()).num_workers(2)
    with pytest.raises(IndexError):
        list(bad)
    bad.close()


def test_samplers():
    s = data.SequentialSampler(5)
    assert s.len() == 5 and list(s) == [0, 1, 2, 3, 4] and s.next_index() is None
    r1, r2 = data.RandomSampler.with_seed(100, 42), data.RandomSampler.with_seed(100, 42)
    l1 = list(r1)
    assert l1 == list(r2) and sorted(l1) == list(range(100)) and l1 != list(range(100))
    r1.reshuffle()
    assert sorted(list(r1)) == list(range(100))
    assert list(data.RandomSampler(50)) != list(data.RandomSampler(50))
    w = data.WeightedRandomSampler([0.0, 1.0, 0.0], 20, seed=1)
    assert w.len() == 20 and set(w) == {1}
    w2 = list(data.WeightedRandomSampler([1.0, 3.0], 4000, seed=2))
    assert 0.70 < sum(w2) / 4000 < 0.80
    with pytest.raises(ValueError):
        data.WeightedRandomSampler([0.0, 0.0], 3)
    b = data.BatchSampler(data.SequentialSampler(7), 3, False)
    assert b.len() == 3 and list(b) == [[0, 1, 2], [3, 4, 5], [6]]
    assert list(data.BatchSampler(data.SequentialSampler(7), 3, True)) == [[0, 1, 2], [3, 4, 5]]
    sub = data.SubsetRandomSampler([3, 5, 7, 9], seed=3)
    assert sorted(sub) == [3, 5, 7, 9]


def test_distributed_sampler_covers_dataset():
    parts = [list(data.DistributedSampler(10, 4, r, shuffle=False)) for r in range(4)]
    assert all(len(p) == 3 for p in parts)  # padded to 12
    assert set(sum(parts, [])) == set(range(10))
    assert parts[0] == [0, 1, 2] and parts[3] == [9, 0, 1]  # wrap-around padding, contiguous rank slices
    sh = [data.DistributedSampler(101, 4, r, shuffle=True, seed=5) for r in range(4)]
    assert set(sum([list(s) for s in sh], [])) == set(range(101))
    e0 = list(data.DistributedSampler(101, 4, 2, True, 5))
    s = data.DistributedSampler(101, 4, 2, True, 5)
    s.set_epoch(1)
    e1 = list(s)
    s.set_epoch(1)
    assert e1 == list(s) and e1 != e0
    with pytest.raises(ValueError):
        data.DistributedSampler(10, 2, 2)


def test_zipf_indices():
    ids = data.zipf_indices(50000, 1.1, 20000, seed=1)
    assert ids.min() >= 0 and ids.max() < 50000
    assert (ids == 0).mean() > 0.05 and (ids < 10).mean() > 0.2
    assert np.array_equal(ids, data.zipf_indices(50000, 1.1, 20000, seed=1))


def test_transforms():
    x = Tensor.from_slice([0.0, 0.5, 1.0])
    assert data.Normalize(0.5, 0.5)(x).to_vec() == pytest.approx([-1, 0, 1])
    assert data.Normalize.standard()(x).to_vec() == x.to_vec()
    assert data.Scale(-1, 1)(x).to_vec() == pytest.approx([-1, 0, 1]) and data.Scale.unit()(x).to_vec() == x.to_vec()
    assert data.Identity()(x) is x
    assert data.Compose([data.Scale.symmetric(), data.Lambda(lambda t: t.mul_scalar(2))])(x).to_vec() == \
        pytest.approx([-2, 0, 2])
    oh = data.ToOneHot(3)(Tensor.from_slice([2, 0], dtype=DType.I64))
    assert oh.to_vec() == [0, 0, 1, 1, 0, 0]
    n = data.GaussianNoise(0.1, seed=0)(Tensor.zeros([1000]))
    assert 0.05 < float(n.torch().std()) < 0.15
    assert data.Normalize.imagenet().mean == 0.485


# ------------------------------------------------------------------------------------- FERRUM01
def _golden():
    """File with two tensors written by hand: 'w' F32 [2,2] = 1..4 at offset 0, 'i' I64 [] = 7 at offset 16."""
    def entry(name, dims, dtype, off, size):
        b = struct.pack("<Q", len(name)) + name.encode()
        b += struct.pack("<Q", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        return b + struct.pack("<IQQ", dtype, off, size)

    header = struct.pack("<IQQQ", 1, 2, 24, 2) + entry("w", [2, 2], 0, 0, 16) + entry("i", [], 5, 16, 8)
    body = struct.pack("<4f", 1, 2, 3, 4) + struct.pack("<q", 7)
    return b"FERRUM01" + struct.pack("<Q", len(header)) + header + body


def test_load_golden_bytes(tmp_path):
    p = tmp_path / "g.ferrum"
    p.write_bytes(_golden())
    t = fb.load(p)
    assert set(t) == {"w", "i"}
    assert t["w"].shape == (2, 2) and t["w"].dtype is DType.F32 and t["w"].to_vec() == [1, 2, 3, 4]
    assert t["i"].shape == () and t["i"].dtype is DType.I64 and t["i"].item() == 7


def test_save_writes_the_reference_layout(tmp_path):
    p = tmp_path / "s.ferrum"
    fb.save({"w": Tensor.from_slice([1.0, 2.0, 3.0, 4.0], [2, 2]), "i": Tensor(torch.tensor(7))}, p)
    assert p.read_bytes() == _golden()


def test_tensors_are_located_by_offset_not_by_map_order(tmp_path):
    def entry(name, dims, dtype, off, size):
        b = struct.pack("<Q", len(name)) + name.encode()
        b += struct.pack("<Q", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        return b + struct.pack("<IQQ", dtype, off, size)

    header = struct.pack("<IQQQ", 1, 2, 12, 2) + entry("late", [2], 4, 4, 8) + entry("early", [1], 0, 0, 4)
    body = struct.pack("<f", 2.5) + struct.pack("<2i", -3, 9)
    p = tmp_path / "o.ferrum"
    p.write_bytes(b"FERRUM01" + struct.pack("<Q", len(header)) + header + body)
    t = fb.load(p)
    assert t["early"].to_vec() == [2.5] and t["late"].to_vec() == [-3, 9] and t["late"].dtype is DType.I32


def test_roundtrip_all_dtypes_and_views(tmp_path):
    src = {
        "f32": Tensor.randn([3, 5]), "f64": Tensor.randn([2], DType.F64), "f16": Tensor.randn([4]).to_dtype(DType.F16),
        "bf16": Tensor.randn([4]).to_dtype(DType.BF16), "i32": Tensor.from_slice([1, -2], dtype=DType.I32),
        "i64": Tensor.arange(4, dtype=DType.I64), "u8": Tensor.from_slice([0, 255], dtype=DType.U8),
        "bool": Tensor(torch.tensor([True, False])), "empty": Tensor.zeros([0, 3]),
        "view": Tensor.arange(6).reshape([2, 3]).t(), "uniçode": Tensor.ones([1]),
    }
    p = tmp_path / "all.ferrum"
    fb.save(src, p)
    out = fb.load(p)
    assert set(out) == set(src)
    for k, v in src.items():
        assert out[k].shape == v.shape and out[k].dtype is v.dtype
        assert torch.equal(out[k].torch(), v.torch().contiguous())


def test_bad_files_raise(tmp_path):
    p = tmp_path / "bad.ferrum"
    p.write_bytes(b"NOTFERRU" + b"\0" * 40)
    with pytest.raises(fb.SerializationError, match="magic"):
        fb.load(p)
    p.write_bytes(b"FERR")
    with pytest.raises(fb.SerializationError):
        fb.load(p)
    p.write_bytes(_golden()[:-4])
    with pytest.raises(fb.SerializationError, match="truncated"):
        fb.load(p)
    with pytest.raises(fb.SerializationError):
        fb.load(tmp_path / "missing.ferrum")
    with pytest.raises(fb.SerializationError):
        fb.save({"c": torch.zeros(2, dtype=torch.complex64)}, tmp_path / "c.ferrum")


def test_corrupt_lengths_in_the_header_are_rejected_not_followed(tmp_path):
    """Lengths an attacker controls (name length, entry count, offset, size) near 2^64 must not wrap the bounds
    checks: every such file is refused with an error, nothing is read outside the data section."""
    def entry(name_len, name, dims, dtype, off, size):
        b = struct.pack("<Q", name_len) + name
        b += struct.pack("<Q", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        return b + struct.pack("<IQQ", dtype, off, size)

    def file(header, body=b"\0" * 24):
        return b"FERRUM01" + struct.pack("<Q", len(header)) + header + body

    big = (1 << 64) - 1
    cases = {
        "name length wraps pos + len": struct.pack("<IQQQ", 1, 1, 24, 1) + entry(big - 7, b"w", [2], 0, 0, 8),
        "entry count far beyond the header": struct.pack("<IQQQ", 1, 1, 24, big // 2) + entry(1, b"w", [2], 0, 0, 8),
        "offset + size wraps": struct.pack("<IQQQ", 1, 1, 24, 1) + entry(1, b"w", [2], 0, big - 3, 8),
        "size beyond the data section": struct.pack("<IQQQ", 1, 1, 24, 1) + entry(1, b"w", [2], 0, 0, 1 << 40),
        "data size wraps data_start + size": struct.pack("<IQQQ", 1, 1, big - 8, 1) + entry(1, b"w", [2], 0, 0, 8),
    }
    p = tmp_path / "evil.ferrum"
    for what, header in cases.items():
        p.write_bytes(file(header))
        with pytest.raises(fb.SerializationError):
            fb.load(p)
    # header length field itself larger than the file
    p.write_bytes(b"FERRUM01" + struct.pack("<Q", big) + b"\0" * 64)
    with pytest.raises(fb.SerializationError):
        fb.load(p)


def test_checkpoint_resume_continues_identically(tmp_path):
    from ferrum_b200 import nn, optim, serialize

    torch.manual_seed(0)
    x, y = Tensor.randn([16, 4]), Tensor.randn([16, 2])

    def make():
        torch.manual_seed(1)
        m = nn.Sequential(nn.Linear(4, 8), nn.Tanh(), nn.Linear(8, 2))
        return m, optim.Adam(m.parameters(), optim.AdamConfig(lr=1e-2)), optim.StepLR(1e-2, 2, 0.5)

    def run(m, o, s, steps):
        out = []
        for _ in range(steps):
            o.set_learning_rate(s.get_lr())
            o.zero_grad()
            l = nn.mse_loss(m(x), y)
            l.backward()
            o.step()
            s.step()
            out.append(l.item())
        return out

    m, o, s = make()
    full = run(m, o, s, 6)
    m, o, s = make()
    first = run(m, o, s, 3)
    serialize.save_checkpoint(tmp_path / "ck.ferrum", m, o, s, extra={"epoch": torch.tensor(3)})
    m2, o2, s2 = make()
    extra = serialize.load_checkpoint(tmp_path / "ck.ferrum", m2, o2, s2)
    assert extra["epoch"].item() == 3 and o2.step_count == 3 and s2.current_step() == 3
    rest = run(m2, o2, s2, 3)
    assert first + rest == pytest.approx(full, rel=1e-6)
    names = set(fb.load(tmp_path / "ck.ferrum"))
    assert {"model.0.weight", "optim.m.0", "optim.v.3", "optim.step", "sched.current_epoch"} <= names
