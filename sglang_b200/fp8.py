"""Weight-side objects of the block-FP8 path: the quantisation config, the linear and MoE
"quant methods" that create / post-process the parameters and call the operators, and a loader for
block-FP8 checkpoints (``weight`` FP8 E4M3 + ``weight_scale_inv`` fp32 per 128x128 block).

They mirror the part of the reference that this path touches
(python/sglang/srt/layers/quantization/fp8.py: ``Fp8Config`` :143-300, ``Fp8LinearMethod``
:309-700 -- ``create_weights`` :397-494, ``process_weights_after_loading_block_quant`` :496-560,
``apply`` -> ``w8a8_block_fp8_linear``; ``Fp8MoEMethod`` :824-1357 -- block-quant branch of
``create_weights`` :980-1060, ``apply`` -> ``fused_experts``), with the same parameter names
(``weight``, ``weight_scale_inv``, ``w13_weight``, ``w13_weight_scale_inv``, ``w2_weight``,
``w2_weight_scale_inv``) so that a state dict of such a checkpoint loads as is. Only what the
block-FP8 path needs is here: dynamic activation scheme, block size [128, 128]; everything else
raises ``NotImplementedError``.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .weight_quant import block_quant_weight_fp8, requant_weight_ue8m0

fp8_dtype = torch.float8_e4m3fn


class Fp8Config:
    """``quantization_config`` of a block-FP8 checkpoint (fp8.py:143-246)."""

    def __init__(self, is_checkpoint_fp8_serialized: bool = False, activation_scheme: str = "dynamic",
                 ignored_layers: Optional[List[str]] = None, weight_block_size: Optional[List[int]] = None):
        if activation_scheme != "dynamic":
            raise NotImplementedError("the block-wise path supports the dynamic activation scheme only")
        if weight_block_size is not None:
            if not is_checkpoint_fp8_serialized:
                raise ValueError("The block-wise quantization only supports fp8-serialized checkpoint for now.")
            if len(weight_block_size) != 2:
                raise ValueError("The quantization block size of weight must have 2 dimensions")
            if list(weight_block_size) != [128, 128]:
                raise NotImplementedError("only weight_block_size [128, 128] is built")
        self.is_checkpoint_fp8_serialized = is_checkpoint_fp8_serialized
        self.activation_scheme = activation_scheme
        self.ignored_layers = ignored_layers or []
        self.weight_block_size = list(weight_block_size) if weight_block_size is not None else [128, 128]

    def get_name(self) -> str:
        return "fp8"

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "Fp8Config":
        quant_method = config["quant_method"]
        ignored = config.get("ignored_layers", config.get("modules_to_not_convert"))
        if ignored:
            normalized = []
            for layer in ignored:
                base = layer.removeprefix("model.")
                normalized += [base, f"model.{base}"]
            ignored = normalized
        return cls(is_checkpoint_fp8_serialized="fp8" in quant_method,
                   activation_scheme=config.get("activation_scheme", "dynamic"), ignored_layers=ignored,
                   weight_block_size=config.get("weight_block_size"))

    def is_layer_skipped(self, prefix: str) -> bool:
        return any(prefix == name or prefix.startswith(name + ".") for name in self.ignored_layers)


def validate_block_quant_shapes(input_size: int, input_size_per_partition: int, output_size: int,
                                output_size_per_partition: int, output_partition_sizes: Sequence[int],
                                tp_size: int, block: Sequence[int] = (128, 128)) -> None:
    """The divisibility rules of the reference (fp8.py:356-395): a row-parallel shard must hold whole
    K blocks, a column-parallel or merged weight whole N blocks per partition."""
    block_n, block_k = block
    if tp_size > 1 and input_size // input_size_per_partition == tp_size:
        if input_size_per_partition % block_k != 0:
            raise ValueError(f"Weight input_size_per_partition = {input_size_per_partition} is not divisible by "
                             f"weight quantization block_k = {block_k}.")
    if (tp_size > 1 and output_size // output_size_per_partition == tp_size) or len(output_partition_sizes) > 1:
        for part in output_partition_sizes:
            if part % block_n != 0:
                raise ValueError(f"Weight output_partition_size = {part} is not divisible by weight quantization "
                                 f"block_n = {block_n}.")


class Fp8LinearMethod:
    """Creates ``weight`` / ``weight_scale_inv`` on a layer and applies the block-FP8 linear."""

    def __init__(self, quant_config: Fp8Config, tp_size: int = 1):
        self.quant_config = quant_config
        self.tp_size = tp_size
        self.block_quant = True

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: List[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, device=None, **extra) -> None:
        out_per_part = sum(output_partition_sizes)
        layer.logical_widths = list(output_partition_sizes)
        layer.input_size_per_partition = input_size_per_partition
        layer.output_size_per_partition = out_per_part
        layer.orig_dtype = params_dtype
        block_n, block_k = self.quant_config.weight_block_size
        validate_block_quant_shapes(input_size, input_size_per_partition, output_size, out_per_part,
                                    output_partition_sizes, self.tp_size, (block_n, block_k))
        serialized = self.quant_config.is_checkpoint_fp8_serialized
        weight = torch.empty(out_per_part, input_size_per_partition, dtype=fp8_dtype if serialized else params_dtype,
                             device=device)
        layer.register_parameter("weight", torch.nn.Parameter(weight, requires_grad=False))
        if serialized:
            scale = torch.full(((out_per_part + block_n - 1) // block_n, (input_size_per_partition + block_k - 1) // block_k),
                               torch.finfo(torch.float32).min, dtype=torch.float32, device=device)
            layer.register_parameter("weight_scale_inv", torch.nn.Parameter(scale, requires_grad=False))

    def process_weights_after_loading(self, layer: torch.nn.Module, requant_ue8m0: bool = False) -> None:
        """A 16-bit checkpoint is block-quantised here; an FP8 checkpoint is taken as loaded
        (fp8.py:496-560). ``requant_ue8m0``: re-quantise to power-of-two scales and pack them for
        MN-major consumers, what the reference does for its DeepGEMM path on Blackwell."""
        if layer.weight.dtype != fp8_dtype:
            q, s = block_quant_weight_fp8(layer.weight.data, self.quant_config.weight_block_size)
            layer.weight = torch.nn.Parameter(q, requires_grad=False)
            layer.register_parameter("weight_scale_inv", torch.nn.Parameter(s, requires_grad=False))
        else:
            assert torch.all(layer.weight_scale_inv.data > torch.finfo(torch.float32).min), "weight_scale_inv not loaded"
        if requant_ue8m0:
            q, s = requant_weight_ue8m0(layer.weight.data, layer.weight_scale_inv.data, self.quant_config.weight_block_size)
            layer.weight = torch.nn.Parameter(q, requires_grad=False)
            layer.weight_scale_inv = torch.nn.Parameter(s.contiguous(), requires_grad=False)
            layer.weight_scale_inv.format_ue8m0 = True

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        from .fp8_kernel import per_token_group_quant_fp8, w8a8_block_fp8_linear, w8a8_block_fp8_matmul

        if getattr(layer.weight_scale_inv, "format_ue8m0", False):
            x2 = x.reshape(-1, x.shape[-1])
            q, s = per_token_group_quant_fp8(x2, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
            out = w8a8_block_fp8_matmul(q, layer.weight, s, layer.weight_scale_inv, [128, 128], output_dtype=x.dtype)
            if bias is not None:
                out = out + bias
            return out.view(*x.shape[:-1], layer.weight.shape[0])
        return w8a8_block_fp8_linear(x, layer.weight, self.quant_config.weight_block_size, layer.weight_scale_inv,
                                     bias=bias)


class Fp8MoEMethod:
    """Creates the stacked expert parameters and applies ``fused_experts`` (fp8.py:824-1357, block-quant
    branch)."""

    def __init__(self, quant_config: Fp8Config):
        self.quant_config = quant_config
        self.block_quant = True

    def create_weights(self, layer: torch.nn.Module, num_experts: int, hidden_size: int,
                       intermediate_size_per_partition: int, params_dtype: torch.dtype, device=None, **extra) -> None:
        block_n, block_k = self.quant_config.weight_block_size
        I, H = intermediate_size_per_partition, hidden_size
        if I % block_n != 0:
            raise ValueError(f"The output_size of gate's and up's weight = {I} is not divisible by weight quantization "
                             f"block_n = {block_n}.")
        serialized = self.quant_config.is_checkpoint_fp8_serialized
        dt = fp8_dtype if serialized else params_dtype
        layer.register_parameter("w13_weight", torch.nn.Parameter(torch.empty(num_experts, 2 * I, H, dtype=dt, device=device), requires_grad=False))
        layer.register_parameter("w2_weight", torch.nn.Parameter(torch.empty(num_experts, H, I, dtype=dt, device=device), requires_grad=False))
        if serialized:
            s13 = torch.ones(num_experts, 2 * ((I + block_n - 1) // block_n), (H + block_k - 1) // block_k, dtype=torch.float32, device=device)
            s2 = torch.ones(num_experts, (H + block_n - 1) // block_n, (I + block_k - 1) // block_k, dtype=torch.float32, device=device)
            layer.register_parameter("w13_weight_scale_inv", torch.nn.Parameter(s13, requires_grad=False))
            layer.register_parameter("w2_weight_scale_inv", torch.nn.Parameter(s2, requires_grad=False))

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        if layer.w13_weight.dtype != fp8_dtype:
            for w_name in ("w13_weight", "w2_weight"):
                q, s = block_quant_weight_fp8(getattr(layer, w_name).data, self.quant_config.weight_block_size)
                setattr(layer, w_name, torch.nn.Parameter(q, requires_grad=False))
                layer.register_parameter(w_name + "_scale_inv", torch.nn.Parameter(s, requires_grad=False))

    def apply(self, layer: torch.nn.Module, hidden_states: torch.Tensor, topk_output, moe_runner_config=None) -> torch.Tensor:
        from .fused_moe import MoeRunnerConfig, fused_experts

        return fused_experts(hidden_states, layer.w13_weight, layer.w2_weight, topk_output,
                             moe_runner_config or MoeRunnerConfig(inplace=False), use_fp8_w8a8=True,
                             w1_scale=layer.w13_weight_scale_inv, w2_scale=layer.w2_weight_scale_inv,
                             block_shape=self.quant_config.weight_block_size)


# ------------------------------------------------------------------------------ checkpoint loader
# Stacked parameters of the model definitions this path serves (the reference's
# ``stacked_params_mapping``, e.g. python/sglang/srt/models/llama.py:560-566, and the expert mapping of
# ``FusedMoE.make_expert_params_mapping``, python/sglang/srt/layers/moe/fused_moe_triton/layer.py).
STACKED_PARAMS = {"q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"),
                  "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}


def _shard(t: torch.Tensor, dim: int, rank: int, size: int, unit: int) -> torch.Tensor:
    """Rank's slice of ``t`` along ``dim`` when the full extent is split evenly in ``unit``-sized elements
    (unit = 1 for a weight, 128 for its block scales: a shard must hold whole blocks)."""
    n = t.shape[dim]
    assert n % size == 0, f"extent {n} (in units of {unit}) does not split over {size} ranks"
    per = n // size
    return t.narrow(dim, rank * per, per)


def load_linear_shard(layer: torch.nn.Module, loaded_weight: torch.Tensor, loaded_scale: torch.Tensor, parallel: str,
                      tp_rank: int, tp_size: int, offset: int = 0) -> None:
    """Copy this rank's part of one checkpoint tensor pair into ``layer.weight[offset:]`` /
    ``layer.weight_scale_inv[offset/128:]``. ``parallel``: "column" (split N), "row" (split K) or
    "replicated". ``offset`` = first output row of a merged parameter (q | k | v, gate | up)."""
    assert parallel in ("column", "row", "replicated")
    if parallel == "column":
        w, s = _shard(loaded_weight, 0, tp_rank, tp_size, 1), _shard(loaded_scale, 0, tp_rank, tp_size, 128)
    elif parallel == "row":
        w, s = _shard(loaded_weight, 1, tp_rank, tp_size, 1), _shard(loaded_scale, 1, tp_rank, tp_size, 128)
    else:
        w, s = loaded_weight, loaded_scale
    n = w.shape[0]
    assert offset % 128 == 0 and (n % 128 == 0 or offset + n == layer.weight.shape[0]), "merged parts hold whole blocks"
    layer.weight.data[offset : offset + n].copy_(w)
    layer.weight_scale_inv.data[offset // 128 : offset // 128 + s.shape[0]].copy_(s)


def load_expert_shard(layer: torch.nn.Module, expert_id: int, shard_id: str, loaded_weight: torch.Tensor,
                      loaded_scale: torch.Tensor, tp_rank: int = 0, tp_size: int = 1) -> None:
    """One expert's ``gate_proj`` ("w1"), ``down_proj`` ("w2") or ``up_proj`` ("w3") pair into the stacked
    parameters; the intermediate dimension is split over ``tp_size`` ranks."""
    assert shard_id in ("w1", "w2", "w3")
    if shard_id == "w2":
        w, s = _shard(loaded_weight, 1, tp_rank, tp_size, 1), _shard(loaded_scale, 1, tp_rank, tp_size, 128)
        layer.w2_weight.data[expert_id].copy_(w)
        layer.w2_weight_scale_inv.data[expert_id].copy_(s)
        return
    w, s = _shard(loaded_weight, 0, tp_rank, tp_size, 1), _shard(loaded_scale, 0, tp_rank, tp_size, 128)
    I = layer.w13_weight.shape[1] // 2
    lo = 0 if shard_id == "w1" else I
    layer.w13_weight.data[expert_id, lo : lo + I].copy_(w)
    layer.w13_weight_scale_inv.data[expert_id, lo // 128 : lo // 128 + s.shape[0]].copy_(s)


def iter_block_fp8_pairs(tensors: Iterable[Tuple[str, torch.Tensor]]):
    """Group an iterable of ``(name, tensor)`` (a safetensors file, a state dict) into
    ``(prefix, weight, weight_scale_inv)`` for every FP8 weight; other tensors come out as
    ``(name, tensor, None)``."""
    pending: Dict[str, Dict[str, torch.Tensor]] = {}
    for name, t in tensors:
        if name.endswith(".weight_scale_inv"):
            key, kind = name[: -len(".weight_scale_inv")], "scale"
        elif name.endswith(".weight") and t.dtype == fp8_dtype:
            key, kind = name[: -len(".weight")], "weight"
        else:
            yield name, t, None
            continue
        slot = pending.setdefault(key, {})
        slot[kind] = t
        if len(slot) == 2:
            del pending[key]
            yield key, slot["weight"], slot["scale"]
    if pending:
        raise ValueError(f"FP8 weights without their scales (or the reverse): {sorted(pending)[:4]}")


def load_safetensors(path: str):
    """``(name, tensor)`` pairs of one ``.safetensors`` file (FP8 tensors included)."""
    from safetensors import safe_open

    with safe_open(path, framework="pt", device="cpu") as f:
        for name in f.keys():
            yield name, f.get_tensor(name)
