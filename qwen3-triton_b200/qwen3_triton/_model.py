"""Qwen3 decoder graph for training, assembled from a parameter table and a set of operator recipes.

The graph is data first: `parameter_table(config)` lists every tensor with its Hugging Face checkpoint name, shape
and initialiser, `plant` hangs them into a tree of plain containers so that `state_dict()` carries exactly those
names, and `DecoderBlock` / `Backbone` / `TritonQwen3ForCausalLM` run the arithmetic through a `Recipe`
(qwen3_triton/components.py) that maps each step - normalise, project, rotate, attend, gate - onto operator-API calls
according to the optimisation switches. One block class therefore serves the plain graph, every ablation variant
and (by overriding `forward`) the fused single-node layer of qwen3_triton/fused.py.

Same contract as the reference graph (qwen3_triton/_model.py:110-134 there): dense, unpadded causal training; no KV
cache, sliding window, attention dropout, RoPE scaling or attention bias - unsupported features raise. The reference
builds one nn.Module subclass per sub-module; only the parameter names, the option names and the forward signature
are shared with it.
"""
from dataclasses import dataclass, fields, replace
from types import SimpleNamespace

import torch
from torch import nn

from . import _abi


# ------------------------------------------------------------------------------------------------ configuration
@dataclass
class Qwen3Config:
    """The subset of the Hugging Face Qwen3 configuration the graph reads (defaults: Qwen3-8B)."""
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False
    model_type: str = 'qwen3'
    hidden_act: str = 'silu'
    attention_dropout: float = 0.0
    attention_bias: bool = False
    use_sliding_window: bool = False
    rope_scaling: object = None


@dataclass(frozen=True)
class ComputeOptions:
    """The reference's three tiling switches (qwen3_triton/_model.py:22-27 there). They select which operator entry
    point a step goes through; the CUDA library picks its own tiles, so results do not depend on them."""
    linear_optimized: bool = False
    attention_optimized: bool = False
    loss_optimized: bool = False


@dataclass(frozen=True)
class OptimizationOptions(ComputeOptions):
    """All switches of the optimised graph (reference qwen3_triton/configuration.py:5-12): the three above default on,
    plus the two fusions and the attention precision switches carried as a tuple of (name, bool) pairs."""
    linear_optimized: bool = True
    attention_optimized: bool = True
    loss_optimized: bool = True
    norm_rope_fusion: bool = True
    mlp_fusion: bool = True
    precision_options: tuple = ()


# variant name -> switches turned off relative to OptimizationOptions(); 'triton_base' is the plain ComputeOptions()
ABLATIONS = {'triton_optimized': (), 'ablate_attention': ('attention_optimized',),
             'ablate_norm_rope': ('norm_rope_fusion',), 'ablate_mlp': ('mlp_fusion',),
             'ablate_linear': ('linear_optimized',), 'ablate_loss': ('loss_optimized',)}
VARIANTS = ('triton_base',) + tuple(ABLATIONS)


def options_for_variant(name):
    if name == 'triton_base':
        return ComputeOptions()
    if name not in ABLATIONS:
        raise ValueError('Unknown Triton variant: ' + str(name))
    return replace(OptimizationOptions(), **{switch: False for switch in ABLATIONS[name]})


def widen_options(options):
    """Any options object -> OptimizationOptions; switches the object does not carry are off."""
    if isinstance(options, OptimizationOptions):
        return options
    names = [f.name for f in fields(OptimizationOptions) if f.name != 'precision_options']
    return OptimizationOptions(**{n: bool(getattr(options, n, False)) for n in names})


def check_config(c):
    if c.model_type != 'qwen3':
        raise ValueError('Official Qwen3 config required')
    if c.hidden_act != 'silu' or c.attention_dropout != 0 or getattr(c, 'attention_bias', False):
        raise ValueError('Only SiLU, zero dropout, bias-free Qwen3 supported')
    if getattr(c, 'use_sliding_window', False) or getattr(c, 'rope_scaling', None):
        raise ValueError('Sliding window and scaled RoPE are not implemented')
    if c.head_dim % 2 or c.num_attention_heads % c.num_key_value_heads:
        raise ValueError('Even rotary dimension and valid GQA required')


# ------------------------------------------------------------------------------------------------ parameter table
def block_table(c):
    """(name inside a decoder layer, shape, initialiser) in the order the forward pass uses them."""
    h, d, i = c.hidden_size, c.head_dim, c.intermediate_size
    q, kv = c.num_attention_heads * d, c.num_key_value_heads * d
    return (('input_layernorm', (h,), 'ones'),
            ('self_attn.q_proj', (q, h), 'normal'), ('self_attn.k_proj', (kv, h), 'normal'),
            ('self_attn.v_proj', (kv, h), 'normal'), ('self_attn.o_proj', (h, q), 'normal'),
            ('self_attn.q_norm', (d,), 'ones'), ('self_attn.k_norm', (d,), 'ones'),
            ('post_attention_layernorm', (h,), 'ones'),
            ('mlp.gate_proj', (i, h), 'normal'), ('mlp.up_proj', (i, h), 'normal'), ('mlp.down_proj', (h, i), 'normal'))


def parameter_table(c):
    """Every parameter of the causal LM: (checkpoint name, shape, initialiser)."""
    rows = [('model.embed_tokens.weight', (c.vocab_size, c.hidden_size), 'normal')]
    for layer in range(c.num_hidden_layers):
        rows += [(f'model.layers.{layer}.{name}.weight', shape, init) for name, shape, init in block_table(c)]
    rows.append(('model.norm.weight', (c.hidden_size,), 'ones'))
    if not c.tie_word_embeddings:
        rows.append(('lm_head.weight', (c.vocab_size, c.hidden_size), 'normal'))
    return rows


class Leaf(nn.Module):
    """One `weight` (matrix: ~N(0, std); vector: ones) and, for norm scales, the epsilon that goes with it."""

    def __init__(self, shape, init, std, eps=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(shape))
        if init == 'ones':
            nn.init.ones_(self.weight)
        else:
            nn.init.normal_(self.weight, std=std)
        self.eps = eps

    def forward(self, op, *inputs):
        """op(*inputs, self), run as this module's forward: wrappers that materialise a module's parameters around
        its call (FSDP units made of a single leaf: token table, final norm) then see the use."""
        return op(*inputs, self)


class Branch(nn.Module):
    """Name-space node of the parameter tree."""


def plant(root, rows, c):
    """Hang a Leaf for every (dotted name, shape, init) row under `root`, creating Branch nodes on the way."""
    for name, shape, init in rows:
        node = root
        *path, last = name.split('.')
        for part in path:
            if not hasattr(node, part):
                node.add_module(part, Branch())
            node = getattr(node, part)
        node.add_module(last, Leaf(shape, init, c.initializer_range, c.rms_norm_eps if init == 'ones' else None))
    return root


def position_ids_for(ids):
    """int64 positions i % S for a [B,S] id tensor, computed on the device."""
    pos = torch.empty(ids.shape, device=ids.device, dtype=torch.int64)
    _abi.call('q3_positions', pos.data_ptr(), ids.numel(), ids.shape[1], _abi.stream())
    return pos


class RotaryTables(nn.Module):
    """inv_freq = theta^(-2i/D) in fp32, turned into cos/sin tables of the activation dtype per call.

    The frequencies are deliberately NOT a registered buffer: `model.to(torch.bfloat16)` would round them to 8 bits
    of mantissa, and a rotation angle is position * frequency - at position 2048 that rounding is an error of
    several radians in the fast components. (The reference keeps them as a buffer and casts back to fp32 at use,
    qwen3_triton/_model.py:49-59 there, which restores the dtype but not the lost bits.) They are built on the CPU
    whatever the default device is, so a meta-device build keeps real values, and copied once per device."""

    def __init__(self, c):
        super().__init__()
        exponent = torch.arange(0, c.head_dim, 2, device='cpu', dtype=torch.float32) / c.head_dim
        self._inv_freq = 1.0 / (c.rope_theta ** exponent)
        self._per_device = {}

    @property
    def inv_freq(self):
        return self._inv_freq

    def frequencies(self, device):
        key = (device.type, device.index)
        if key not in self._per_device:
            self._per_device[key] = self._inv_freq.to(device)
        return self._per_device[key]

    def forward(self, positions, dtype):
        from .kernels.rotary import rotary_tables
        return rotary_tables(positions, self.frequencies(positions.device), dtype)


# ------------------------------------------------------------------------------------------------ graph
class DecoderBlock(nn.Module):
    """Pre-norm attention + gated MLP with residuals; parameters from block_table, arithmetic from the recipe."""

    def __init__(self, c, recipe):
        super().__init__()
        plant(self, [(name, shape, init) for name, shape, init in block_table(c)], c)
        self.recipe = recipe
        self.heads, self.kv_heads, self.head_dim = c.num_attention_heads, c.num_key_value_heads, c.head_dim

    def attention(self, x, rope):
        r, a = self.recipe, self.self_attn
        b, s, _ = x.shape
        q = r.project(x, a.q_proj).view(b, s, self.heads, self.head_dim)
        k = r.project(x, a.k_proj).view(b, s, self.kv_heads, self.head_dim)
        v = r.project(x, a.v_proj).view(b, s, self.kv_heads, self.head_dim)
        q, k = r.normalise_and_rotate(q, a.q_norm, rope), r.normalise_and_rotate(k, a.k_norm, rope)
        y = r.attend(*(t.transpose(1, 2).contiguous() for t in (q, k, v)))          # [B, heads, S, D]
        return r.project(y.transpose(1, 2).contiguous().view(b, s, self.heads * self.head_dim), a.o_proj)

    def forward(self, x, rope):
        r = self.recipe
        x = r.add(x, self.attention(r.normalise(x, self.input_layernorm), rope))
        return r.add(x, r.gated_mlp(r.normalise(x, self.post_attention_layernorm), self.mlp))


class Backbone(nn.Module):
    """embed -> blocks -> final norm. `block_class` is the only thing the fused variant changes."""
    block_class = DecoderBlock

    def __init__(self, c, recipe):
        super().__init__()
        plant(self, [('embed_tokens', (c.vocab_size, c.hidden_size), 'normal')], c)
        self.layers = nn.ModuleList(self.block_class(c, recipe) for _ in range(c.num_hidden_layers))
        plant(self, [('norm', (c.hidden_size,), 'ones')], c)
        self.rotary_emb = RotaryTables(c)
        self.recipe = recipe

    def lookup(self, ids):
        # embed_tokens is a Leaf, or a module with its own forward when the table is sharded by vocabulary rows
        if isinstance(self.embed_tokens, Leaf):
            return self.embed_tokens(self.recipe.embed, ids)
        return self.embed_tokens(ids)

    def rope_for(self, ids, position_ids, dtype):
        if position_ids is None:
            position_ids = position_ids_for(ids)
        elif position_ids.shape == (1, ids.shape[1]) and ids.shape[0] != 1:
            position_ids = position_ids.expand(ids.shape[0], -1).contiguous()
        if position_ids.shape != ids.shape:
            raise ValueError('position_ids must match batch and sequence')
        return self.rotary_emb(position_ids, dtype)

    def forward(self, ids, position_ids=None):
        x = self.lookup(ids)
        rope = self.rope_for(ids, position_ids, x.dtype)
        for block in self.layers:
            x = block(x, rope)
        return self.norm(self.recipe.normalise, x)


_UNSUPPORTED = ('use_cache', 'attention_mask', 'past_key_values', 'output_attentions', 'output_hidden_states',
                'logits_to_keep')


class TritonQwen3ForCausalLM(nn.Module):
    """Causal LM over the graph above. `forward(input_ids, labels)` returns an object with `.loss` and `.logits`.

    `lm_head` is a Leaf (logits = hidden W^T, then the shifted cross-entropy), or any module that maps
    (hidden, labels) to (loss, logits-or-None) itself - the vocabulary-parallel head does, and with it the
    [tokens, vocab] logits never exist."""
    backbone_class = Backbone

    def __init__(self, config, options=None):
        super().__init__()
        from .components import Recipe
        check_config(config)
        self.config = config
        self.options = options or ComputeOptions()
        self.model = self.backbone_class(config, Recipe(self.options))
        if config.tie_word_embeddings:
            self.lm_head = Branch()
        else:
            plant(self, [('lm_head', (config.vocab_size, config.hidden_size), 'normal')], config)
        self.tie_weights()

    def tie_weights(self):
        if self.config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def load_hf_state_dict(self, state, *, assign=False):
        """Strict load of a Hugging Face Qwen3 state dict (a tied checkpoint may omit lm_head.weight)."""
        state = dict(state)
        if self.config.tie_word_embeddings:
            table = state['model.embed_tokens.weight']
            if not torch.equal(state.setdefault('lm_head.weight', table), table):
                raise ValueError('Checkpoint disagrees with tied embedding configuration')
        result = self.load_state_dict(state, strict=True, assign=assign)
        self.tie_weights()
        return result

    def load_safetensors(self, *files, assign=False):
        """Load a Hugging Face checkpoint stored as one or more .safetensors shards."""
        from .checkpoint import read_safetensors
        state = {}
        for path in files:
            state.update(read_safetensors(path))
        return self.load_hf_state_dict(state, assign=assign)

    def forward(self, input_ids, labels=None, *, position_ids=None, return_dict=True, diagnostic_logits=False, **extra):
        unknown = set(extra) - set(_UNSUPPORTED)
        if unknown:
            raise TypeError('Unexpected arguments: ' + ', '.join(sorted(unknown)))
        if any(extra.get(k) not in (None, False, 0) for k in _UNSUPPORTED):
            raise ValueError('Only dense unpadded causal training without cache/extra outputs is implemented; no fallback')
        if input_ids.ndim != 2 or input_ids.dtype not in (torch.int32, torch.int64):
            raise ValueError('Integer [B,S] input_ids required')
        hidden = self.model(input_ids, position_ids)
        head = self.lm_head
        if not isinstance(head, (Leaf, Branch)):
            if labels is None:
                raise ValueError('Vocabulary CE requires dense unpadded labeled loss-only training/evaluation')
            loss, logits = head(hidden, labels, diagnostics=diagnostic_logits)
            return SimpleNamespace(loss=loss, logits=logits) if return_dict else (loss, logits)
        recipe = self.model.recipe
        logits = recipe.project(hidden, head)
        loss = recipe.loss(logits, labels) if labels is not None else None
        if return_dict:
            return SimpleNamespace(loss=loss, logits=logits)
        return (logits,) if labels is None else (loss, logits)
