"""The dependency-free safetensors reader against the safetensors package's own writer and reader, and the model's
`load_safetensors` path (two shards, strict names)."""
import pytest
import torch

import recipe


def test_reader_matches_the_safetensors_package(tmp_path):
    from qwen3_triton.checkpoint import read_safetensors, write_safetensors
    st = pytest.importorskip('safetensors.torch')
    g = torch.Generator().manual_seed(0)
    tensors = {'a.weight': torch.randn(5, 7, generator=g).to(torch.bfloat16), 'b': torch.randn(3, generator=g),
               'ids': torch.arange(11, dtype=torch.int64), 'h': torch.randn(2, 2, 2, generator=g).to(torch.float16),
               'empty': torch.empty(0, 4)}
    theirs, ours = tmp_path / 'theirs.safetensors', tmp_path / 'ours.safetensors'
    st.save_file(tensors, str(theirs), metadata={'format': 'pt'})
    write_safetensors(ours, tensors)
    for source in (read_safetensors(theirs), read_safetensors(ours), st.load_file(str(ours))):
        assert set(source) == set(tensors)
        for name, t in tensors.items():
            assert source[name].dtype == t.dtype and torch.equal(source[name], t), name
    assert set(read_safetensors(theirs, names={'b'})) == {'b'}
    bad = tmp_path / 'bad.safetensors'
    bad.write_bytes(b'\x01\x02')
    with pytest.raises(ValueError):
        read_safetensors(bad)


def test_model_loads_sharded_safetensors(tmp_path):
    from qwen3_triton import model_for_variant
    from qwen3_triton.checkpoint import write_safetensors
    c = recipe.tiny_config()
    state = recipe.seeded_state(c)
    names = sorted(state)
    write_safetensors(tmp_path / 'model-00001-of-00002.safetensors', {n: state[n] for n in names[:10]})
    write_safetensors(tmp_path / 'model-00002-of-00002.safetensors', {n: state[n] for n in names[10:]})
    model = model_for_variant(c, 'triton_optimized')
    model.load_safetensors(*sorted(tmp_path.glob('*.safetensors')))
    for n, p in model.named_parameters():
        assert torch.equal(p.detach(), state[n]), n
    with pytest.raises(RuntimeError):
        model_for_variant(c, 'triton_optimized').load_safetensors(tmp_path / 'model-00001-of-00002.safetensors')
