"""Data path and validation partition on the CPU: the oracle restatement (oracle/data.py) and the package's host
classes (training/data.py, training/evaluation.py) against fixtures produced by the reference's own code
(tests/golden/data.npz, written by tests/golden/make_golden.py), plus the reference's known-answer cases
(its tests/test_data.py:9-27 and tests/test_evaluation.py:7-26) restated on this package."""
import math

import numpy as np
import pytest
import torch

from oracle import data as OD


@pytest.fixture(scope='module')
def golden_data():
    from conftest import ROOT
    data = np.load(ROOT / 'tests' / 'golden' / 'data.npz')
    return {k: data[k] for k in data.files}


def corpus_cases(golden):
    case = 0
    while f'data{case}/meta' in golden:
        yield case, [int(v) for v in golden[f'data{case}/meta']]
        case += 1


def test_oracle_reproduces_reference_block_order(golden_data):
    for case, (tokens, seq, seed, offset, blocks, stride) in corpus_cases(golden_data):
        assert tokens // seq == blocks
        assert OD.stride_for(blocks) == stride and math.gcd(stride, blocks) == 1
        firsts = golden_data[f'data{case}/train_first_tokens']
        order = OD.block_order(blocks, len(firsts), seed=seed, offset=offset)
        assert [b * seq for b in order] == firsts.tolist()          # token value == position in these corpora
        wrap = OD.block_order(blocks, 4, seed=seed, offset=offset, first=blocks)
        assert [b * seq for b in wrap] == golden_data[f'data{case}/wrap_first_tokens'].tolist()


def test_package_blocks_reproduce_reference(golden_data, tmp_path):
    from training.data import Blocks, coprime_stride
    for case, (tokens, seq, seed, offset, blocks, stride) in corpus_cases(golden_data):
        path = tmp_path / f'c{case}.bin'
        np.arange(tokens, dtype='<u4').tofile(path)
        train, plain = Blocks(path, seq, offset=offset, training=True, seed=seed), Blocks(path, seq)
        assert len(train) == blocks and train.stride == stride == coprime_stride(blocks)
        firsts = golden_data[f'data{case}/train_first_tokens']
        assert [int(train[i][0]) for i in range(len(firsts))] == firsts.tolist()
        assert [int(train[blocks + i][0]) for i in range(4)] == golden_data[f'data{case}/wrap_first_tokens'].tolist()
        last = plain[blocks - 1]
        assert last.dtype == torch.int64 and last.tolist() == golden_data[f'data{case}/eval_last_block'].tolist()
        assert torch.equal(train[3], OD.read_block(np.arange(tokens, dtype='<u4'), seq, train.block_index(3)))


def test_blocks_known_answers(tmp_path):
    """51 tokens in blocks of 5: ten blocks, tail dropped; file order for evaluation; the training order is a
    permutation of all ten given by (i * stride + seed) mod 10."""
    from training.data import Blocks
    path = tmp_path / 'corpus.bin'
    np.arange(51, dtype='<u4').tofile(path)
    plain, train = Blocks(path, 5), Blocks(path, 5, training=True, seed=42)
    assert len(plain) == 10
    for i in range(10):
        assert plain[i].tolist() == list(range(5 * i, 5 * i + 5))
        assert torch.equal(train[i], plain[(i * train.stride + 42) % 10])
    assert len({tuple(train[i].tolist()) for i in range(10)}) == 10
    for bad in (0, 1, -1, 2.5):
        with pytest.raises(ValueError):
            Blocks(tmp_path / 'missing.bin', bad)
    short = tmp_path / 'short.bin'
    np.arange(3, dtype='<u4').tofile(short)
    with pytest.raises(ValueError):
        Blocks(short, 5)


def test_validation_partition_and_nll_reproduce_reference(golden_data):
    from training.evaluation import shifted_nll, validation_batches
    case = 0
    while f'val{case}/meta' in golden_data:
        size, world, batch = (int(v) for v in golden_data[f'val{case}/meta'])
        ids, table = torch.from_numpy(golden_data[f'val{case}/ids']), torch.from_numpy(golden_data[f'val{case}/table'])
        masks, served, total, count, forwards = [], [], 0.0, 0, []
        oracle_total, oracle_count = 0.0, 0
        for rank in range(world):
            calls = 0
            plan = OD.partition(size, rank, world, batch)
            for call, (data, valid) in enumerate(validation_batches(list(ids), rank, world, batch)):
                assert [i is not None for i in plan[call]] == valid.tolist()
                assert torch.equal(data, torch.stack([ids[i if i is not None else 0] for i in plan[call]]))
                logits = torch.stack([table[i if i is not None else 0] for i in plan[call]])
                n, c = shifted_nll(logits, data, valid)
                on, oc = OD.shifted_nll(logits, data, valid)
                total, count = total + float(n), count + int(c)
                oracle_total, oracle_count = oracle_total + on, oracle_count + oc
                masks.append(valid.numpy())
                served.append(data.numpy())
                calls += 1
            forwards.append(calls)
        assert len(set(forwards)) == 1                                  # same number of forwards on every rank
        assert np.array_equal(np.stack(masks), golden_data[f'val{case}/valid'])
        assert np.array_equal(np.stack(served), golden_data[f'val{case}/served'])
        ref_total, ref_count = golden_data[f'val{case}/total_count']
        assert count == oracle_count == int(ref_count) == size * 5
        assert total == pytest.approx(float(ref_total), rel=1e-6) and oracle_total == pytest.approx(float(ref_total), rel=1e-6)
        full = torch.nn.functional.cross_entropy(table[:, :-1].reshape(-1, 11), ids[:, 1:].reshape(-1), reduction='sum')
        assert total == pytest.approx(float(full), rel=1e-6)             # == the unpartitioned loss
        case += 1
    assert case >= 4
    for bad in ((-1, 1, 1), (2, 2, 1), (0, 0, 1), (0, 1, 0)):
        with pytest.raises(ValueError):
            next(validation_batches([torch.zeros(3)], *bad))
    with pytest.raises(ValueError):
        next(validation_batches([], 0, 1, 1))
