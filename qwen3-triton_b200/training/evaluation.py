"""Exact validation over every block of a dataset, partitioned over data ranks.

Semantics of the reference's training/evaluation.py:7-47. Every rank runs the same number of forwards of the same
shape (so collectives inside the model line up): the blocks are dealt out in rounds of world*batch, rank r taking the
r-th group of `batch`; positions past the end of the dataset re-use block 0 as input and are masked out of the loss.
The summed negative log-likelihood and the token count travel as two fp64 numbers on the device, one all-reduce at the
end, and the count must equal blocks * (seq - 1) exactly or the result is refused.

The arithmetic runs in the CUDA library: per-row losses from the shifted cross-entropy kernel (q3_ce_fwd), their fp64
sum and count from q3_validation_rows; a model that returns only a loss (vocabulary-parallel head) contributes
loss * tokens through qwen3_triton.runtime.metrics.accumulate_validation.
"""
import torch
import torch.distributed as dist

IGNORE = -100


def validation_batches(dataset, rank, world, batch):
    """Yields (ids [batch, seq], valid [batch] bool) for this rank; the same number of items on every rank."""
    size = len(dataset)
    if world < 1 or batch < 1 or not 0 <= rank < world or size < 1:
        raise ValueError('Invalid validation partition')
    per_round = world * batch
    rounds = -(-size // per_round)
    for r in range(rounds):
        first = r * per_round + rank * batch
        wanted = range(first, first + batch)
        valid = torch.tensor([i < size for i in wanted], dtype=torch.bool)
        ids = torch.stack([dataset[i if i < size else 0] for i in wanted])
        yield ids, valid


def masked_labels(ids, valid):
    """Labels equal to the ids, with every position of an invalid (padding) block set to ignore."""
    return torch.where(valid.to(ids.device)[:, None], ids, torch.full_like(ids, IGNORE))


def shifted_nll(logits, ids, valid):
    """(summed NLL of token t+1 given logits at t over the valid blocks, number of scored tokens). CUDA logits go
    through the library's kernels and come back as fp64 scalars on the device; CPU tensors (tests of the partition
    logic) use the same definition in torch."""
    if logits.ndim != 3 or ids.shape != logits.shape[:2] or valid.shape != ids.shape[:1]:
        raise ValueError('Expected logits [B,S,V], ids [B,S] and valid [B]')
    labels = masked_labels(ids, valid)
    if not logits.is_cuda:
        rows = logits[:, :-1].float().reshape(-1, logits.shape[-1])
        total = torch.nn.functional.cross_entropy(rows, labels[:, 1:].reshape(-1), ignore_index=IGNORE, reduction='sum')
        return total, valid.sum() * (ids.shape[1] - 1)
    from qwen3_triton import _abi
    b, s, v = logits.shape
    dev = logits.device
    logits, labels = logits.contiguous(), labels.contiguous()
    n = b * (s - 1)
    lse, target, losses = (torch.empty(n, device=dev, dtype=torch.float32) for _ in range(3))
    mean = torch.empty((), device=dev, dtype=torch.float32)
    count = torch.empty((), device=dev, dtype=torch.int32)
    totals = torch.zeros(2, device=dev, dtype=torch.float64)
    word = torch.zeros(1, device=dev, dtype=torch.int32)   # a batch of padding only has no target: not an error here
    _abi.call('q3_ce_fwd', logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), target.data_ptr(), losses.data_ptr(),
              mean.data_ptr(), count.data_ptr(), b, s, v, IGNORE, _abi.dt(logits.dtype), word.data_ptr(), _abi.stream())
    _abi.call('q3_validation_rows', losses.data_ptr(), labels.data_ptr(), b, s, IGNORE, totals.data_ptr(), _abi.stream())
    return totals[0], totals[1]


@torch.no_grad()
def evaluate_full(model, dataset, batch=4, *, device='cuda'):
    """Token-mean loss over the whole dataset: dict(loss, tokens, blocks). Works without a process group (one rank)."""
    from qwen3_triton.runtime.metrics import accumulate_validation
    distributed = dist.is_available() and dist.is_initialized()
    rank, world = (dist.get_rank(), dist.get_world_size()) if distributed else (0, 1)
    was_training = model.training
    model.eval()
    totals = torch.zeros(2, device=device, dtype=torch.float64)
    seq = None
    try:
        for ids, valid in validation_batches(dataset, rank, world, batch):
            seq = ids.shape[1]
            ids = ids.to(device)
            out = model(ids, labels=masked_labels(ids, valid), use_cache=False)
            if getattr(out, 'logits', None) is not None:
                nll, count = shifted_nll(out.logits, ids, valid)
                totals += torch.stack([nll.double(), count.double()])
            else:
                accumulate_validation(totals, out.loss, int(valid.sum()) * (seq - 1))
        if distributed:
            dist.all_reduce(totals)
        expected = len(dataset) * (seq - 1)
        nll, count = totals.tolist()
        if count != expected:
            raise RuntimeError('Validation token coverage mismatch')
        if not (nll == nll and abs(nll) != float('inf')) or expected == 0:
            raise RuntimeError('Invalid validation loss')
        return dict(loss=nll / count, tokens=expected, blocks=len(dataset))
    finally:
        model.train(was_training)
