"""``torch.ops.humming.*``: the operator-level surface of the reference, on the C ABI.

The reference exposes its launcher as two dispatcher operators, and frameworks
that embed it (or trace it with ``torch.compile``) call those rather than
``HummingLayer``:

* ``humming::launch_humming`` (``humming/csrc/launcher/launcher.cpp:220-224``), the
  GEMM itself, dense and indexed (MoE);
* ``humming::humming_quant_input`` (``humming/kernel/quant_input.py:144-150``), the
  per-token activation quantizer that precedes an FP8-activation GEMM.

Both are defined here with the reference's schema, argument for argument, a
CUDA implementation that goes through :mod:`humming_b200.runtime` (pointers and
the current stream into the native library), and a fake implementation that
computes output shapes and dtypes only, so that tracing works.  There is no CPU
implementation: calling either operator on CPU tensors fails in the dispatcher.

Two arguments carry a different payload from the reference's, because there is
no table of JIT-compiled kernels to index here:

``configs``
    The reference passes ``(min_m, max_m, kernel_id)`` triples.  Here it is the
    layer descriptor as integers -- the fields of ``hm_gemm_desc`` in declaration
    order (``include/humming_b200.h``), see :func:`desc_to_configs` -- optionally
    followed by ``(min_m, max_m, token_tile)`` triples that pick the token tile by
    the number of rows, like ``HummingMethod.add_kernel_config``.
``locks``
    The reference's lock words (int32[1024], zero on entry).  Here the layer's
    workspace: any tensor of at least ``hm_gemm_workspace_bytes`` /
    ``hm_moe_gemm_workspace_bytes`` bytes, zero-filled once by the caller.  The
    operator never allocates one, and refuses a missing or short workspace.

``register_kernel`` (``launcher.cpp:225``) has no counterpart: nothing is compiled
or loaded at run time.
"""
from typing import List, Optional, Sequence, Tuple

import torch

from humming_b200 import dtypes
from humming_b200 import native
from humming_b200 import runtime

LAUNCH_SCHEMA = (
    "(int[] configs, Tensor a, Tensor b, Tensor(c!)? c, Tensor? as_, Tensor? bs, Tensor? bzp, Tensor? bias, "
    "Tensor? gs, Tensor? topk_weights, Tensor? sorted_token_ids, Tensor? expert_ids, "
    "Tensor? num_tokens_post_padded, Tensor(locks!)? locks, int num_ctas_per_sm=1, int? num_sms=None, "
    "bool should_check_tensor=True) -> Tensor")
QUANT_SCHEMA = "(Tensor inputs, str dtype, Tensor? scales=None, int? group_size=None) -> (Tensor, Tensor)"

_DESC_FIELDS = [name for name, _ in native.GemmDesc._fields_]
_NATIVE_TO_TORCH = {1: torch.float16, 2: torch.bfloat16, 3: torch.float32, 4: torch.float8_e4m3fn,
                    5: torch.float8_e5m2, 6: torch.float8_e8m0fnu}

_lib = torch.library.Library("humming", "FRAGMENT")
_lib.define("launch_humming" + LAUNCH_SCHEMA)
_lib.define("humming_quant_input" + QUANT_SCHEMA)


def desc_to_configs(desc: native.GemmDesc, tile_table: Sequence[int] = ()) -> List[int]:
    """``configs`` for :func:`launch_humming`: the descriptor's fields, then the
    ``(min_m, max_m, token_tile)`` triples (may be empty: the plan picks the tile)."""
    if len(tile_table) % 3:
        raise ValueError("the token-tile table is a flat list of (min_m, max_m, token_tile) triples")
    return [int(getattr(desc, name)) for name in _DESC_FIELDS] + [int(v) for v in tile_table]


def layer_configs(layer, sublayer_name: str = "") -> List[int]:
    """``configs`` of one (sub)layer built by ``HummingMethod``: its descriptor with the options given to
    ``prepare_default_kernel_configs`` / ``add_kernel_config`` (``top_k``, ``is_moe_down``, ``use_stream_k``,
    ``native_flags``) and its token-tile table -- what ``HummingMethod.forward_layer`` derives per call.  The
    counterpart of the reference's generated ``get_kernel_configs`` module (``humming/layer.py:489-499``)."""
    from humming_b200.layer import HummingMethod

    meta = layer.humming_metas[sublayer_name]
    opts = layer.humming_kernel_options[sublayer_name]
    flags = (0 if opts.get("use_stream_k", True) else native.HM_FLAG_NO_SPLIT_K) | opts.get("native_flags", 0)
    desc = HummingMethod._desc(meta, top_k=opts.get("top_k", 0), is_moe_down=bool(opts.get("is_moe_down", False)),
                               flags=flags)
    return desc_to_configs(desc, layer.humming_block_size_configs[sublayer_name])


def configs_to_desc(configs: Sequence[int], m: int) -> native.GemmDesc:
    """Inverse of :func:`desc_to_configs` for a call with ``m`` rows."""
    nf = len(_DESC_FIELDS)
    if len(configs) < nf or (len(configs) - nf) % 3:
        raise ValueError(f"configs must hold {nf} descriptor fields followed by (min_m, max_m, token_tile) triples, "
                         f"got {len(configs)} integers")
    desc = native.GemmDesc(**{name: int(v) for name, v in zip(_DESC_FIELDS, configs)})
    for i in range(nf, len(configs), 3):
        if configs[i] <= m <= configs[i + 1]:
            desc.m_tile = int(configs[i + 2])
            break
    return desc


def _output_sizes(configs: Sequence[int], a: torch.Tensor) -> Tuple[List[int], torch.dtype]:
    """Shape and dtype of ``c`` when the caller passes none (``humming/csrc/launcher/tensor.h:9-20``): the
    leading sizes of ``a``, ``top_k`` appended for an MoE up projection, then N."""
    desc = configs_to_desc(configs, 0)
    sizes = list(a.shape[:-1])
    if desc.num_experts and not desc.is_moe_down:
        sizes.append(desc.top_k)
    sizes.append(desc.shape_n)
    return sizes, _NATIVE_TO_TORCH[desc.c_dtype]


def _launch_fake(configs, a, b, c=None, as_=None, bs=None, bzp=None, bias=None, gs=None, topk_weights=None,
                 sorted_token_ids=None, expert_ids=None, num_tokens_post_padded=None, locks=None, num_ctas_per_sm=1,
                 num_sms=None, should_check_tensor=True):
    if c is not None:
        return c
    sizes, dtype = _output_sizes(configs, a)
    return a.new_empty(sizes, dtype=dtype)


def _rows(t: torch.Tensor) -> torch.Tensor:
    t = t.reshape(-1, t.size(-1))
    if t.stride(-1) != 1 or (t.stride(0) * t.element_size()) % 16 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def _launch_cuda(configs, a, b, c=None, as_=None, bs=None, bzp=None, bias=None, gs=None, topk_weights=None,
                 sorted_token_ids=None, expert_ids=None, num_tokens_post_padded=None, locks=None, num_ctas_per_sm=1,
                 num_sms=None, should_check_tensor=True):
    if gs is not None:
        raise NotImplementedError("a global scale is not built")
    if locks is None:
        raise ValueError("launch_humming needs the layer's workspace in `locks` (it never allocates one)")
    rows = _rows(a)
    desc = configs_to_desc(configs, rows.size(0))
    if desc.num_experts and desc.is_moe_down and desc.top_k:
        # MoE tables are keyed by tokens; a down projection sees top_k rows per token
        desc = configs_to_desc(configs, rows.size(0) // desc.top_k)
    if num_sms is not None:
        desc.num_sms = int(num_sms)
    moe = desc.num_experts > 0
    if moe and desc.flags & (native.HM_FLAG_MOE_A_SORTED | native.HM_FLAG_MOE_C_SORTED):
        # those layouts need the token count as a separate argument, which this schema has no place for
        raise NotImplementedError("pre-sorted MoE activations / outputs are reached through HummingLayer.forward "
                                  "(inputs_sorted / outputs_sorted), not through launch_humming")
    if should_check_tensor:
        if rows.size(1) != desc.shape_k:
            raise ValueError(f"a has K={rows.size(1)}, the descriptor says {desc.shape_k}")
        if rows.dtype != _NATIVE_TO_TORCH.get(desc.a_dtype):
            raise ValueError(f"a is {rows.dtype}, the descriptor says {_NATIVE_TO_TORCH.get(desc.a_dtype)}")
        if (desc.a_dtype == 4) != (as_ is not None):
            raise ValueError("as_ (one fp32 scale per row of a) goes with FP8 activations, and only with them")
        if moe and (sorted_token_ids is None or expert_ids is None or num_tokens_post_padded is None):
            raise ValueError("an MoE descriptor needs sorted_token_ids, expert_ids and num_tokens_post_padded")
        if not moe and sorted_token_ids is not None:
            raise ValueError("routing tensors given to a dense descriptor")
        if moe and desc.is_moe_down and topk_weights is None:
            raise ValueError("the down projection needs topk_weights")
    sizes, c_dtype = _output_sizes(configs, a)
    if c is None:
        c = torch.empty(sizes, dtype=c_dtype, device=a.device)
    elif should_check_tensor:
        if c.dtype != c_dtype or not c.is_contiguous() or c.numel() != _numel(sizes):
            raise ValueError(f"c must be a contiguous {c_dtype} tensor of {sizes}")
    if c.numel() == 0:
        return c
    if as_ is not None:
        as_ = as_.reshape(-1).float().contiguous()
        if should_check_tensor and as_.numel() != rows.size(0):
            raise ValueError("as_ must hold one fp32 scale per row of a")
    out = c.view(-1, desc.shape_n)
    if not moe:
        runtime.gemm(desc, rows, b, bs, bzp, bias, out, locks, a_scale=as_)
        return c
    num_valid = rows.size(0) * (1 if desc.is_moe_down else desc.top_k)
    ids = sorted_token_ids if sorted_token_ids.dtype == torch.int32 else sorted_token_ids.int()
    tkw = None if topk_weights is None else topk_weights.reshape(-1).float().contiguous()
    runtime.moe_gemm(desc, num_valid, rows, b, bs, bzp, bias, tkw, ids.contiguous(), expert_ids.int().contiguous(),
                     num_tokens_post_padded.reshape(-1).int(), out, locks, a_scale=as_)
    return c


def _numel(sizes) -> int:
    n = 1
    for s in sizes:
        n *= int(s)
    return n


def _quant_shapes(inputs, dtype, scales, group_size):
    if dtypes.DataType.from_str(dtype) != dtypes.float8e4m3:
        raise NotImplementedError(f"activation quantization to {dtype} is not built")
    if scales is not None:
        raise NotImplementedError("static activation scales are not built: pass scales=None (dynamic, per token)")
    if group_size not in (None, 0, inputs.size(-1)):
        raise NotImplementedError("grouped activation scales are not built: one scale per token only")


def _quant_fake(inputs, dtype, scales=None, group_size=None):
    _quant_shapes(inputs, dtype, scales, group_size)
    rows = _numel(inputs.shape[:-1])
    return (torch.empty_like(inputs, dtype=torch.float8_e4m3fn),
            inputs.new_empty((rows, 1), dtype=torch.float32))


def _quant_cuda(inputs, dtype, scales=None, group_size=None):
    _quant_shapes(inputs, dtype, scales, group_size)
    q, s = runtime.quant_input(inputs, dtype)
    return q, s.reshape(-1, 1)    # the reference returns (rows, groups) scales, groups = 1 per token


_lib.impl("launch_humming", _launch_cuda, "CUDA")
_lib.impl("humming_quant_input", _quant_cuda, "CUDA")
torch.library.register_fake("humming::launch_humming", _launch_fake, lib=_lib)
torch.library.register_fake("humming::humming_quant_input", _quant_fake, lib=_lib)

launch_humming = torch.ops.humming.launch_humming
humming_quant_input = torch.ops.humming.humming_quant_input


def workspace_bytes(configs: Sequence[int], m: int, capacity: Optional[int] = None) -> int:
    """Bytes ``locks`` must hold for a call with ``m`` rows (dense) or a ``sorted_token_ids`` of ``capacity``
    entries (MoE)."""
    desc = configs_to_desc(configs, m)
    if desc.num_experts:
        if capacity is None:
            raise ValueError("an MoE descriptor needs the capacity of sorted_token_ids")
        return runtime.moe_workspace_bytes(desc, capacity)
    return runtime.workspace_bytes(desc, m)
