"""Reading Hugging Face checkpoints stored as .safetensors shards, without any dependency beyond torch.

A .safetensors file is: 8 bytes little-endian header length n, n bytes of JSON mapping tensor name ->
{"dtype", "shape", "data_offsets": [begin, end]} (plus an optional "__metadata__" entry), then the raw little-endian
tensor bytes, offsets relative to the end of the header. The file is memory-mapped, so a 16 GB checkpoint costs no
host copy until a tensor is moved to the GPU.
"""
import json
import mmap
import struct

import torch

_DTYPES = {'F64': torch.float64, 'F32': torch.float32, 'F16': torch.float16, 'BF16': torch.bfloat16,
           'I64': torch.int64, 'I32': torch.int32, 'I16': torch.int16, 'I8': torch.int8, 'U8': torch.uint8,
           'BOOL': torch.bool}


def read_safetensors(path, *, names=None):
    """{name: tensor} for one shard; `names` restricts it to a subset. Tensors are views of a read-only memory map:
    copy (`.clone()`, `.to(device)`) before writing to them."""
    with open(path, 'rb') as fh:
        head = fh.read(8)
        if len(head) != 8:
            raise ValueError('Not a safetensors file: shorter than its length field')
        (length,) = struct.unpack('<Q', head)
        header = json.loads(fh.read(length).decode('utf-8'))
        mapped = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
    base = 8 + length
    out = {}
    for name, entry in header.items():
        if name == '__metadata__' or (names is not None and name not in names):
            continue
        dtype = _DTYPES.get(entry['dtype'])
        if dtype is None:
            raise ValueError(f"Unsupported safetensors dtype {entry['dtype']} for {name}")
        begin, end = entry['data_offsets']
        count = 1
        for dim in entry['shape']:
            count *= dim
        if end - begin != count * torch.empty((), dtype=dtype).element_size():
            raise ValueError(f'Corrupt entry for {name}: byte range does not match shape and dtype')
        if count == 0:
            out[name] = torch.empty(entry['shape'], dtype=dtype)
            continue
        flat = torch.frombuffer(mapped, dtype=dtype, count=count, offset=base + begin)
        out[name] = flat.view(entry['shape'])
    return out


def write_safetensors(path, tensors):
    """Inverse of read_safetensors for CPU tensors (used by the tests and for exporting small states)."""
    names = {v: k for k, v in _DTYPES.items()}
    header, blobs, offset = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b''
        header[name] = {'dtype': names[t.dtype], 'shape': list(t.shape), 'data_offsets': [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    text = json.dumps(header, separators=(',', ':')).encode('utf-8')
    text += b' ' * (-len(text) % 8)                 # keep the data 8-byte aligned
    with open(path, 'wb') as fh:
        fh.write(struct.pack('<Q', len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw)
