"""GPU parity of the device-side partitioner against a numpy/scipy restatement of the reference's
(partition/distchunk_manager.py:63-157, examples/dist_gcn/dist_partition.py:122-158)."""
import numpy as np
import pytest
import torch

from test_partition_cpu import make_partitioned, reference_chunks

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("n,E,P", [(500, 6000, 4), (64, 300, 1), (3000, 50000, 8)])
def test_partition_to_chunks(cuda, tmp_path, n, E, P):
    from jittorgeometric_b200.partition import DistChunk, chunks_save, distributed_file, partition_to_chunks
    partition, edge_index, w = make_partitioned(n + P, n, E, P)
    rng = np.random.default_rng(3)
    feature = rng.standard_normal((n, 7)).astype(np.float32)
    label = rng.integers(0, 5, size=n).astype(np.int64)
    masks = [rng.random(n) < 0.5, rng.random(n) < 0.2, None]
    chunks = partition_to_chunks(partition, dev(edge_index.astype(np.int32)), n, P, dev(w), dev(feature),
                                 [dev(masks[0]), dev(masks[1]), None], dev(label), num_classes=5)
    ref = reference_chunks(partition, edge_index, n, P, w)
    assert len(chunks) == P
    for p, (c, r) in enumerate(zip(chunks, ref)):
        s, e = r["range"]
        assert (c.chunks, c.chunk_id, c.v_num, c.global_v_num, c.num_classes) == (P, p, e - s, n, 5)
        assert np.array_equal(host(c.offset), r["offset"])
        assert np.array_equal(host(c.edge_index), r["edge_index"]) and np.array_equal(host(c.edge_weight), r["edge_weight"])
        assert np.array_equal(host(c.CSR.row_offset), r["csr"].indptr) and np.array_equal(host(c.CSR.column_indices), r["csr"].indices)
        assert np.array_equal(host(c.CSR.edge_weight), r["csr"].data)
        assert np.array_equal(host(c.CSC.column_offset), r["csc"].indptr) and np.array_equal(host(c.CSC.row_indices), r["csc"].indices)
        assert np.array_equal(host(c.CSC.edge_weight), r["csc"].data)
        order = r["order"]
        assert np.array_equal(host(c.local_feature), feature[order][s:e]) and np.array_equal(host(c.local_label), label[order][s:e])
        assert np.array_equal(host(c.local_masks["train"]), masks[0][order][s:e]) and c.local_masks["test"] is None
        for q in range(P):
            lo, hi = r["offset"][q], r["offset"][q + 1]
            blk = r["csr"][lo:hi]
            assert np.array_equal(host(c.chunk_CSR[q].row_offset), blk.indptr)
            assert np.array_equal(host(c.chunk_CSR[q].column_indices), blk.indices)
            assert np.array_equal(host(c.chunk_CSR[q].edge_weight), blk.data)
    # device chunks -> disk -> device
    chunks_save(chunks, str(tmp_path))
    back = DistChunk.load(distributed_file(P - 1, P, str(tmp_path)), device="cuda")
    assert torch.equal(back.CSC.row_indices, chunks[-1].CSC.row_indices) and back.CSC.row_indices.is_cuda
    assert torch.equal(back.local_feature, chunks[-1].local_feature)
    assert torch.equal(back.chunk_CSR[0].column_indices, chunks[-1].chunk_CSR[0].column_indices)


def test_partition_with_an_empty_part(cuda):
    """A part that owns no node gives a chunk with no rows and no entries; the others are unaffected."""
    from jittorgeometric_b200.partition import partition_to_chunks
    n, P = 40, 3
    rng = np.random.default_rng(2)
    pairs = np.unique(rng.integers(0, n, size=(300, 2)), axis=0).T
    partition = np.where(rng.random(n) < 0.5, 0, 2).astype(np.int32)      # nobody in part 1
    w = rng.random(pairs.shape[1]).astype(np.float32)
    chunks = partition_to_chunks(partition, dev(pairs.astype(np.int32)), n, P, dev(w))
    ref = reference_chunks(partition, pairs, n, P, w)
    assert chunks[1].v_num == 0 and chunks[1].CSC.row_indices.numel() == 0 and host(chunks[1].CSC.column_offset).tolist() == [0]
    for c, r in zip(chunks, ref):
        assert np.array_equal(host(c.CSC.column_offset), r["csc"].indptr) and np.array_equal(host(c.CSC.row_indices), r["csc"].indices)
        assert np.array_equal(host(c.CSR.row_offset), r["csr"].indptr) and np.array_equal(host(c.CSR.column_indices), r["csr"].indices)
