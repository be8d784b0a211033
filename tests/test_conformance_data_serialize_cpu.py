"""Per-symbol behaviour checks of ``ferrotorch_b200.data`` (samplers, dataset combinators, transforms, array bridges, loader modes) and of
the GGUF / safetensors records of ``ferrotorch_b200.serialize``."""
import struct

import numpy as np
import pytest
import torch

import ferrotorch_b200.data as D
import ferrotorch_b200.serialize as S


def test_samplers():
    s = D.SequentialSampler(5)
    assert isinstance(s, D.Sampler) and s.indices() == [0, 1, 2, 3, 4] and len(s) == 5 and list(s) == [0, 1, 2, 3, 4]
    r = D.RandomSampler(10, seed=3)
    a, b = r.indices(0), r.indices(1)
    assert sorted(a) == list(range(10)) and a != b and r.indices(0) == a                 # a permutation per epoch, reproducible
    rr = D.RandomSampler(4, seed=1, replacement=True, num_samples=50)
    assert len(rr.indices()) == 50 and set(rr.indices()) <= {0, 1, 2, 3}
    w = D.WeightedRandomSampler([0.0, 1.0, 3.0], 4000, seed=0)
    idx = torch.tensor(w.indices())
    assert (idx == 0).sum() == 0 and 2.5 < (idx == 2).sum().item() / max(1, (idx == 1).sum().item()) < 3.6
    bs = D.BatchSampler(D.SequentialSampler(7), 3)
    assert bs.batches() == [[0, 1, 2], [3, 4, 5], [6]] and len(bs) == 3
    assert D.BatchSampler(D.SequentialSampler(7), 3, drop_last=True).batches() == [[0, 1, 2], [3, 4, 5]]


def test_dataset_combinators_and_streams():
    base = D.VecDataset([1, 2, 3])
    m = D.MappedDataset(base, lambda v: v * 10)
    assert len(m) == 3 and [m[i] for i in range(3)] == [10, 20, 30]

    class Count(D.IterableDataset):
        def __init__(self, lo, hi):
            self.lo, self.hi = lo, hi

        def iter(self, worker_info=None):
            wi = worker_info or D.WorkerInfo(0, 1)
            return iter(range(self.lo + wi.worker_id, self.hi, wi.num_workers))

    ch = D.ChainDataset([Count(0, 3), Count(10, 12)])
    assert list(ch) == [0, 1, 2, 10, 11]
    assert list(ch.iter(D.WorkerInfo(1, 2))) == [1, 11]
    info = D.WorkerInfo(worker_id=1, num_workers=4, seed=7)
    assert (info.worker_id, info.num_workers, info.seed) == (1, 4, 7)
    tok = D.SyntheticTokenDataset(8, seq_len=16, vocab=100, seed=1)
    assert len(tok) == 8 and tok[3].shape == (17,) and torch.equal(tok[3], tok[3]) and not torch.equal(tok[3], tok[4]) and int(tok[3].max()) < 100


def test_collate_transforms_and_loader_modes():
    batch = D.default_collate([(torch.ones(2), 1), (torch.zeros(2), 0)])
    assert batch[0].shape == (2, 2) and batch[1].tolist() == [1, 0]
    d = D.default_collate([{"x": torch.ones(1), "y": 2.0}, {"x": torch.zeros(1), "y": 3.0}])
    assert d["x"].shape == (2, 1) and d["y"].tolist() == [2.0, 3.0]
    img = torch.arange(12.0).view(3, 2, 2)
    n = D.Normalize([1.0, 2.0, 3.0], [2.0, 2.0, 2.0])(img)
    assert torch.allclose(n[1], (img[1] - 2.0) / 2.0)
    assert D.ToFloat()(torch.tensor([1, 2])).dtype == torch.float32
    assert D.Lambda(lambda t: t + 1)(torch.zeros(1)).item() == 1.0
    td = D.ToDevice("cpu")
    assert td.device == "cpu" and td.non_blocking
    assert {m.value for m in D.WorkerMode} == {"sync", "threads"}
    ds = D.TensorDataset(torch.arange(10.0).view(10, 1), torch.arange(10))
    for cls in (D.CollatedIter, D.PrefetchIter, D.MultiWorkerIter):
        ld = cls(ds, batch_size=4, num_workers=2 if cls is D.MultiWorkerIter else 0, prefetch=2)
        got = torch.cat([b[1] for b in ld])
        assert got.tolist() == list(range(10)) and len(ld) == 3


def test_array_bridges(tmp_path):
    t = torch.arange(6, dtype=torch.float32).view(2, 3)
    a = D.to_numpy(t)
    assert isinstance(a, np.ndarray) and a.shape == (2, 3) and a[1, 2] == 5
    p = tmp_path / "t.npy"
    D.save_npy(str(p), t)
    assert torch.equal(D.load_npy(str(p)), t) and np.array_equal(np.load(p), a)
    pa = pytest.importorskip("pyarrow")
    assert D.from_arrow(pa.array([1.5, 2.5, 3.5])).tolist() == [1.5, 2.5, 3.5]
    assert D.from_arrow(pa.chunked_array([[1, 2], [3]])).tolist() == [1, 2, 3]


def _gguf_bytes():
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    w = np.arange(64, dtype=np.float32).reshape(2, 32)
    kv = s("general.architecture") + struct.pack("<I", 8) + s("llama")
    ti = s("w") + struct.pack("<I", 2) + struct.pack("<QQ", 32, 2) + struct.pack("<I", 0) + struct.pack("<Q", 0)
    head = b"GGUF" + struct.pack("<I", 3) + struct.pack("<QQ", 1, 1) + kv + ti
    head += b"\0" * (-len(head) % 32)
    return head + w.tobytes(), w


def test_gguf_records_and_mapped_loading(tmp_path):
    img, w = _gguf_bytes()
    p = tmp_path / "m.gguf"
    p.write_bytes(img)
    g = S.load_gguf_mmap(p)
    assert isinstance(g, S.GgufData) and isinstance(g.metadata, S.GgufMetadata) and g.version == 3
    t = g.tensors[0]
    assert isinstance(t, S.GgufTensor) and t.name == "w" and tuple(t.dims) in ((32, 2), (2, 32))
    assert torch.equal(S.dequantize_gguf_tensor(g, "w"), torch.from_numpy(w))
    f = S.parse_gguf(p)
    assert isinstance(f, S.GgufFile) and isinstance(f.tensors["w"], S.GgufTensorInfo) and f.tensors["w"].ggml_type == 0
    assert f.metadata["general.architecture"] == "llama" and f.data_offset % 32 == 0


def test_safetensors_metadata_mapped_loading_and_shard_progress(tmp_path):
    a, b = torch.arange(6.0).view(2, 3), torch.ones(4, dtype=torch.bfloat16)
    p = tmp_path / "x.safetensors"
    S.save_safetensors({"a": a, "b": b}, p)
    meta = S.safetensors_metadata(p)
    assert meta["a"]["shape"] == [2, 3] and meta["a"]["dtype"] == "F32" and meta["b"]["dtype"] == "BF16"
    m = S.load_safetensors_mmap(p)
    assert torch.equal(m["a"], a) and torch.equal(m["b"], b)
    S.save_safetensors({"a": a}, tmp_path / "s1.safetensors")
    S.save_safetensors({"b": b}, tmp_path / "s2.safetensors")
    import json
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    seen = []
    sd = S.load_safetensors_sharded_with_progress(tmp_path / "model.safetensors.index.json", seen.append)
    assert torch.equal(sd["a"], a) and len(seen) == 2 and all(isinstance(e, S.ShardProgress) for e in seen)
    assert [e.shard_index for e in seen] == [0, 1] and seen[0].shard_count == 2 and seen[-1].total_tensors == 2
    assert seen[1].tensors_loaded_so_far == 1


def test_default_collate_keeps_named_tuples_lists_and_dicts():
    from typing import NamedTuple
    import ferrotorch_b200.data as D

    class Sample(NamedTuple):
        image: torch.Tensor
        label: int
    batch = D.default_collate([Sample(torch.full((2, 2), float(i)), i) for i in range(3)])
    assert isinstance(batch, Sample) and batch.image.shape == (3, 2, 2) and batch.label.tolist() == [0, 1, 2]
    pair = D.default_collate([(torch.zeros(2), 1.5), (torch.ones(2), 2.5)])
    assert isinstance(pair, tuple) and pair[0].shape == (2, 2) and pair[1].tolist() == [1.5, 2.5]
    lst = D.default_collate([[1, 2], [3, 4]])
    assert isinstance(lst, list) and lst[0].tolist() == [1, 3]
    dct = D.default_collate([{"a": torch.zeros(1)}, {"a": torch.ones(1)}])
    assert dct["a"].shape == (2, 1)
