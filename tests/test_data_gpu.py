"""Device side of the data path and of validation: bit-exact block order and token gather from a corpus resident in
GPU memory, fp64 validation accumulators, and a full-coverage evaluation of a tiny model against the oracle model."""
import numpy as np
import pytest
import torch

import recipe
from oracle import data as OD
from oracle.model import OracleQwen3

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('tokens,seq,seed,offset', [(51, 5, 42, 0), (100003, 7, 20261102, 11), (4096 * 33 + 5, 2048, 3, 2)])
def test_device_blocks_are_bit_identical_to_host_blocks(tmp_path, tokens, seq, seed, offset):
    from qwen3_triton import _abi
    from training.data import Blocks, DeviceBlocks
    path = tmp_path / 'corpus.bin'
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 2 ** 32, size=tokens, dtype=np.uint64).astype('<u4')   # includes ids >= 2^31
    raw.tofile(path)
    for training in (True, False):
        host = Blocks(path, seq, offset=offset, training=training, seed=seed)
        dev = DeviceBlocks(host)
        n = len(host)
        count = min(n, 9)
        first = 0 if not training else n - 3          # crosses the wrap-around in training order
        expect_order = OD.block_order(n, count, seed=seed, offset=offset, training=training, first=first)
        assert dev.order(first, count).tolist() == expect_order
        ids = dev.batch(first, count)
        assert ids.dtype == torch.int64 and ids.shape == (count, seq)
        expect = torch.stack([OD.read_block(raw, seq, b) for b in expect_order])
        assert torch.equal(ids.cpu(), expect)
        if training or first + count <= n:
            assert torch.equal(ids.cpu(), torch.stack([host[first + i] for i in range(count)]))
    assert _abi.read_status() == 0


def test_block_order_is_exact_beyond_64_bit_products():
    from qwen3_triton import _abi
    out = torch.empty(5, device='cuda', dtype=torch.int64)
    first, offset, stride, seed, n = 2 ** 40, 2 ** 41 + 7, 2 ** 31 - 1, 2 ** 62 + 12345, 2 ** 45 - 55
    _abi.call('q3_block_order', out.data_ptr(), first, 5, offset, stride, seed, n, 1, _abi.stream())
    assert out.tolist() == [((first + i + offset) * stride + seed) % n for i in range(5)]


def test_out_of_range_block_sets_status_and_is_not_read():
    from qwen3_triton import _abi
    corpus = torch.arange(40, device='cuda', dtype=torch.int32)
    index = torch.tensor([1, 9, -1], device='cuda', dtype=torch.int64)       # 4 blocks of 10: 9 and -1 are outside
    ids = torch.full((3, 10), -7, device='cuda', dtype=torch.int64)
    word = torch.zeros(1, device='cuda', dtype=torch.int32)
    _abi.call('q3_token_blocks', corpus.data_ptr(), 40, index.data_ptr(), ids.data_ptr(), 3, 10, word.data_ptr(), _abi.stream())
    assert int(word.item()) == _abi.STATUS_ID_RANGE
    assert ids[0].tolist() == list(range(10, 20)) and ids[1:].abs().sum().item() == 0


def test_validation_accumulators_match_fp64_host_arithmetic():
    from qwen3_triton.runtime.metrics import accumulate_validation
    from training.evaluation import shifted_nll
    totals = torch.zeros(2, device='cuda', dtype=torch.float64)
    expect = [0.0, 0.0]
    for value, tokens in ((2.7182817, 8188), (11.931, 0), (0.33333334, 123457), (9.5, 1)):
        loss = torch.tensor(value, device='cuda', dtype=torch.float32)
        accumulate_validation(totals, loss, tokens)
        expect = OD.accumulate(expect, value, tokens) if tokens else expect
    assert totals.tolist() == expect                                          # bit-identical fp64
    with pytest.raises(ValueError):
        accumulate_validation(totals.float(), loss, 1)
    with pytest.raises(ValueError):
        accumulate_validation(totals, loss, -1)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 300, (5, 33), generator=g)
    logits = (torch.randn(5, 33, 300, generator=g) * 2).to(torch.bfloat16)
    valid = torch.tensor([True, False, True, True, False])
    nll, count = shifted_nll(logits.cuda(), ids.cuda(), valid)
    ref_nll, ref_count = OD.shifted_nll(logits.float(), ids, valid)
    assert int(count.item()) == ref_count == 3 * 32
    assert abs(float(nll) - ref_nll) / ref_nll < 1e-5
    none_nll, none_count = shifted_nll(logits.cuda(), ids.cuda(), torch.zeros(5, dtype=torch.bool))
    assert float(none_nll) == 0.0 and float(none_count) == 0.0


@pytest.mark.parametrize('variant', ['triton_optimized', 'b200_fused'])
def test_full_coverage_evaluation_matches_oracle_model(tmp_path, variant):
    """17 blocks, batches of 4: the last forward carries three padding blocks. Loss over exactly 17 * (seq-1) tokens
    equals the oracle model's summed NLL / tokens."""
    from types import SimpleNamespace
    from qwen3_triton import model_for_variant
    from training.data import Blocks
    from training.evaluation import evaluate_full
    c = recipe.tiny_config()
    if variant == 'b200_fused':
        c = SimpleNamespace(**{**vars(c), **dict(head_dim=128, num_attention_heads=2, num_key_value_heads=1)})
    seq, blocks = 48, 17
    rng = np.random.default_rng(5)
    raw = rng.integers(0, c.vocab_size, size=seq * blocks + 11).astype('<u4')
    path = tmp_path / 'val.bin'
    raw.tofile(path)
    data = Blocks(path, seq)
    state = {k: v.to(torch.bfloat16).float() for k, v in recipe.seeded_state(c, seed=9).items()}
    model = model_for_variant(c, variant)
    model.load_hf_state_dict({k: v.clone() for k, v in state.items()})
    model = model.to('cuda', torch.bfloat16)
    result = evaluate_full(model, data, batch=4)
    assert result['tokens'] == blocks * (seq - 1) and result['blocks'] == blocks and model.training
    oracle = OracleQwen3(c, state=state)
    total = 0.0
    with torch.no_grad():
        for i in range(blocks):
            ids = data[i][None]
            loss, _ = oracle(ids, ids)
            total += float(loss) * (seq - 1)
    assert abs(result['loss'] - total / (blocks * (seq - 1))) / result['loss'] < 2e-3
