"""Drop-in Pairformer modules backed by the b200pf CUDA kernels.

Call surface mirrors the reference:
  * ``B200PairformerModule(token_s, token_z, num_blocks, num_heads=16, dropout=0.25,
    pairwise_head_width=32, pairwise_num_heads=4, post_layer_norm=False,
    activation_checkpointing=False, v2=False, **kw).forward(s, z, mask, pair_mask,
    use_kernels=False) -> (s, z)``            (tt_bio/reference.py:921-1003)
  * ``B200PairformerNoSeqModule(token_z, num_blocks, ...).forward(z, pair_mask,
    use_kernels=False) -> z``                 (tt_bio/reference.py:1096-1139)
  * ``B200PairformerLayer.forward(s, z, mask, pair_mask, chunk_size_tri_attn=None,
    use_kernels=False, ...)``                 (tt_bio/reference.py:865-914)
  * ``B200PairformerNoSeqLayer(token_z, ...).forward(z, pair_mask, chunk_size_tri_attn=None,
    use_kernels=False, ...) -> z``            (tt_bio/reference.py:1007-1095)
  * the device backend's constructor, which is what the template / confidence / affinity / Protenix /
    ESMFold2 call sites build: ``B200PairformerModule(n_blocks, tri_att_head_dim, tri_att_n_heads,
    att_head_dim, att_n_heads, transform_s, affinity=False).forward(s or None, z, mask=None,
    pair_mask=None, use_kernels=False) -> (s or None, z)``   (tt_bio/tenstorrent.py:2194-2234,
    tt_bio/boltz2.py:3751, 4503, 4689, 5016)
Parameters carry the reference's state-dict key names, so ``load_state_dict`` of a reference
checkpoint slice works unchanged (tt_bio/tenstorrent.py:2179-2180 does the same for its backend).

Inference only (eval-mode semantics: dropout masks are 1).  Inputs must be CUDA tensors; there
is no CPU path.  The fused kernels are built for c_z = 128 with 4 x 32 triangle-attention heads (Boltz-2's trunk, MSA
and confidence stacks); other widths (the template stack's c_z = 64, the c_z = 256 / 8-head trunks of sibling models)
run on the un-fused fp32 kernels, which take any width: pass ``precision="fp32"`` or ``"auto"``.
``precision``: "bf16" (fused tensor-core kernels, fp32 residual stream),
"mxfp8" (as bf16, but the triangle-multiplication operands a / b are MXFP8: e4m3 values with one
e8m0 scale per 32 elements along the contraction index, contracted by the block-scaled tensor-core
instruction - the counterpart of the reference's block-fp8 fast mode, tt_bio/tenstorrent.py:178-181)
or "fp32" (un-fused fp32 kernels, the validation tier).
"""
from __future__ import annotations

import os
import re
from typing import Dict, Optional, Tuple

import torch
from torch import nn

from . import ops, weights
from .synthetic import layer_param_shapes


def _register_tree(root: nn.Module, name: str, shape) -> None:
    parts = name.split(".")
    mod = root
    for p in parts[:-1]:
        if p not in mod._modules:
            mod.add_module(p, nn.Module())
        mod = mod._modules[p]
    mod.register_parameter(parts[-1], nn.Parameter(torch.zeros(shape), requires_grad=False))


def _mask_u8(m: Optional[torch.Tensor], shape, device) -> torch.Tensor:
    if m is None:
        return torch.ones(shape, dtype=torch.uint8, device=device)
    return (m.reshape(shape) != 0).to(device=device, dtype=torch.uint8).contiguous()


class SideTrack:
    """The stream the single track runs on, beside the pair track.

    The single track of block b needs z after block b's pair transition and s after block b-1, and nothing in the
    pair track ever reads s: so it can run on a stream of its own, under the next block's pair kernels (and, in the
    sharded trunk, under its exchanges, which leave most SMs idle).  Its one read of z, the pair-bias projection,
    has to be over before the next block first writes z: ``bias_read`` is the event the pair stream waits for
    at that point."""

    def __init__(self, device: torch.device) -> None:
        self.stream = torch.cuda.Stream(device)
        self.bias_read: Optional[torch.cuda.Event] = None

    def mark_z_read(self) -> None:
        self.bias_read = torch.cuda.Event()
        self.bias_read.record()

    def before_z_write(self) -> None:
        if self.bias_read is not None:
            torch.cuda.current_stream().wait_event(self.bias_read)
            self.bias_read = None

    def join(self) -> None:
        torch.cuda.current_stream().wait_stream(self.stream)
        self.bias_read = None


class B200PairformerLayer(nn.Module):
    """One Pairformer block (with or without the single track)."""

    def __init__(self, token_s: int = 384, token_z: int = 128, num_heads: int = 16, dropout: float = 0.25,
                 pairwise_head_width: int = 32, pairwise_num_heads: int = 4, post_layer_norm: bool = False,
                 v2: bool = False, precision: str = "bf16", with_s: bool = True) -> None:
        super().__init__()
        if post_layer_norm:
            raise NotImplementedError("post_layer_norm=True is not used by Boltz-2 and is not built")
        if precision == "auto":     # the fused kernels where their widths fit, the un-fused fp32 kernels elsewhere
            precision = "bf16" if (token_z, pairwise_num_heads, pairwise_head_width) == (128, 4, 32) else "fp32"
        if precision not in ("bf16", "mxfp8", "fp32"):
            raise ValueError("precision must be 'bf16', 'mxfp8', 'fp32' or 'auto'")
        self.token_s, self.token_z, self.num_heads = token_s, token_z, num_heads
        self.dropout, self.with_s, self.precision = dropout, with_s, precision
        self.fused = precision != "fp32"
        self.mx_contract_variant = 2   # 2 = block-scaled tcgen05, 0 = expand to bf16 + bf16 contraction (cross-check)
        for name, shape in layer_param_shapes(token_s, token_z, num_heads, pairwise_num_heads,
                                              pairwise_head_width, with_s):
            _register_tree(self, name, shape)
        self._packed: Optional[Dict[str, Dict[str, torch.Tensor]]] = None
        self.register_load_state_dict_post_hook(lambda module, incompatible: module.reset_static_cache())
        self._register_load_state_dict_pre_hook(_accept_backend_keys)

    # same name as the reference backend's cache reset (tt_bio/tenstorrent.py:2185-2191)
    def reset_static_cache(self) -> None:
        self._packed = None

    def _pack(self, device) -> Dict[str, Dict[str, torch.Tensor]]:
        if self._packed is not None and self._packed["_device"] == device:
            return self._packed
        sd = {k: v for k, v in self.state_dict().items()}
        pk: Dict[str, Dict[str, torch.Tensor]] = {"_device": device}
        for name in ("tri_mul_out", "tri_mul_in"):
            pk[name] = (weights.pack_trimul(sd, name + ".", device) if self.fused
                        else weights.to_device_f32(sd, name + ".", device))
        for name in ("tri_att_start", "tri_att_end"):
            pk[name] = (weights.pack_triatt(sd, name + ".", device) if self.fused
                        else weights.to_device_f32(sd, name + ".", device))
        pk["transition_z"] = (weights.pack_transition_z(sd, "transition_z.", device) if self.fused
                              else weights.to_device_f32(sd, "transition_z.", device))
        if self.with_s:
            pk["pre_norm_s"] = weights.to_device_f32(sd, "pre_norm_s.", device)
            pk["attention"] = weights.to_device_f32(sd, "attention.", device)
            pk["transition_s"] = weights.to_device_f32(sd, "transition_s.", device)
            pk["s_fused"] = ops.pack_single_track(pk["attention"], pk["transition_s"])
        self._packed = pk
        return pk

    def forward_inplace(self, s: Optional[torch.Tensor], z: torch.Tensor, tok_mask_u8: Optional[torch.Tensor],
                        masks: ops.PairMasks, ws: Optional[ops.Workspace], side: Optional["SideTrack"] = None) -> None:
        """Update fp32 working copies z [N,N,128] and s [N,c_s] in place.  With a ``side`` track the update of s is
        only enqueued on its stream (the caller joins it before reading s)."""
        pk = self._pack(z.device)
        wait_bias = side.before_z_write if side is not None else None
        if self.fused:
            if self.precision == "mxfp8":
                ops.tri_mul_mxfp8(z, masks.pm, pk["tri_mul_out"], ws, False, self.mx_contract_variant, wait_bias)
                ops.tri_mul_mxfp8(z, masks.pm, pk["tri_mul_in"], ws, True, self.mx_contract_variant)
            else:
                ops.tri_mul_bf16(z, masks.pm, pk["tri_mul_out"], ws, False, wait_bias)
                ops.tri_mul_bf16(z, masks.pm, pk["tri_mul_in"], ws, True)
            ops.tri_att_bf16(z, masks, pk["tri_att_start"], ws, False)
            ops.tri_att_bf16(z, masks, pk["tri_att_end"], ws, True)
            ops.transition_z_bf16(z, pk["transition_z"])
        else:
            if side is not None:
                side.before_z_write()
            ops.tri_mul_f32(z, masks.pm, pk["tri_mul_out"], False)
            ops.tri_mul_f32(z, masks.pm, pk["tri_mul_in"], True)
            ops.tri_att_f32(z, masks.pm, pk["tri_att_start"], False)
            ops.tri_att_f32(z, masks.pm, pk["tri_att_end"], True)
            ops.transition_f32(z, pk["transition_z"])
        if self.with_s and s is not None:
            if side is None:
                ops.single_track(s, z, tok_mask_u8, pk["pre_norm_s"], pk["attention"], pk["transition_s"], self.num_heads,
                                 pk["s_fused"])
            else:
                z_ready = torch.cuda.Event()
                z_ready.record()
                with torch.cuda.stream(side.stream):
                    side.stream.wait_event(z_ready)
                    ops.single_track(s, z, tok_mask_u8, pk["pre_norm_s"], pk["attention"], pk["transition_s"], self.num_heads,
                                     pk["s_fused"], side.mark_z_read)

    def forward(self, s: Optional[torch.Tensor], z: torch.Tensor, mask: Optional[torch.Tensor] = None,
                pair_mask: Optional[torch.Tensor] = None, chunk_size_tri_attn: Optional[int] = None,
                use_kernels: bool = False, use_cuequiv_mul: bool = False, use_cuequiv_attn: bool = False
                ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        return _run_layers([self], s, z, mask, pair_mask)


class B200PairformerNoSeqLayer(B200PairformerLayer):
    """Pair-only block with the reference's constructor and ``forward(z, pair_mask, ...) -> z``
    (tt_bio/reference.py:1007-1095)."""

    def __init__(self, token_z: int = 128, dropout: float = 0.25, pairwise_head_width: int = 32,
                 pairwise_num_heads: int = 4, post_layer_norm: bool = False, precision: str = "bf16") -> None:
        super().__init__(384, token_z, 16, dropout, pairwise_head_width, pairwise_num_heads, post_layer_norm,
                         False, precision, with_s=False)

    def forward(self, z: torch.Tensor, pair_mask: Optional[torch.Tensor] = None,      # type: ignore[override]
                chunk_size_tri_attn: Optional[int] = None, use_kernels: bool = False,
                use_cuequiv_mul: bool = False, use_cuequiv_attn: bool = False) -> torch.Tensor:
        return _run_layers([self], None, z, None, pair_mask)[1]


class B200PairUpdateBlock(nn.Module):
    """The block of the ESMFold2 folding trunk (tt_bio/esmfold2.py:129-154): ``z += tri_mul_out(z); z += tri_mul_in(z);
    z += transition(z)``, no triangle attention, any pair width and transition width.  Keys as in the Pairformer layer
    (``tri_mul_out.*``, ``tri_mul_in.*``, ``transition_z.*``); ``remaps.esmfold2_pair_update_block`` produces them from
    an ESMFold2 checkpoint.  Runs on the un-fused fp32 kernels."""

    def __init__(self, token_z: int = 256, hidden: Optional[int] = None) -> None:
        super().__init__()
        hidden = hidden or 4 * token_z
        self.token_z, self.hidden = token_z, hidden
        for name in ("tri_mul_out", "tri_mul_in"):
            for leaf, shape in (("norm_in.weight", (token_z,)), ("norm_in.bias", (token_z,)),
                                ("p_in.weight", (2 * token_z, token_z)), ("g_in.weight", (2 * token_z, token_z)),
                                ("norm_out.weight", (token_z,)), ("norm_out.bias", (token_z,)),
                                ("p_out.weight", (token_z, token_z)), ("g_out.weight", (token_z, token_z))):
                _register_tree(self, f"{name}.{leaf}", shape)
        for leaf, shape in (("norm.weight", (token_z,)), ("norm.bias", (token_z,)), ("fc1.weight", (hidden, token_z)),
                            ("fc2.weight", (hidden, token_z)), ("fc3.weight", (token_z, hidden))):
            _register_tree(self, f"transition_z.{leaf}", shape)
        self._packed = None
        self.register_load_state_dict_post_hook(lambda module, incompatible: setattr(module, "_packed", None))

    def _pack(self, device):
        if self._packed is None or self._packed["_device"] != device:
            sd = dict(self.state_dict().items())
            self._packed = {"_device": device}
            for name in ("tri_mul_out", "tri_mul_in", "transition_z"):
                self._packed[name] = weights.to_device_f32(sd, name + ".", device)
        return self._packed

    def forward_inplace(self, z: torch.Tensor, pair_mask_u8: torch.Tensor) -> None:
        """z [N, N, c_z] contiguous fp32, updated where it is; pair_mask_u8 [N, N]."""
        pk = self._pack(z.device)
        ops.tri_mul_f32(z, pair_mask_u8, pk["tri_mul_out"], False)
        ops.tri_mul_f32(z, pair_mask_u8, pk["tri_mul_in"], True)
        ops.transition_f32(z, pk["transition_z"])

    def forward(self, z: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """z [1, N, N, c_z], mask [1, N, N] or None -> z."""
        if not z.is_cuda:
            raise RuntimeError("B200 Pairformer: inputs must be CUDA tensors (there is no CPU path)")
        n = z.shape[1]
        with torch.cuda.device(z.device), torch.no_grad():
            zw = z[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
            self.forward_inplace(zw, _mask_u8(mask, (n, n), z.device))
        return zw[None]


_TRI_ATT_KEY = re.compile(r"((?:^|\.)tri_att_(?:start|end)\.)linear_[qkvog]\.")


def _accept_backend_keys(state_dict, prefix, *_unused) -> None:
    """The reference's device backend reads the triangle-attention projections with or without the
    ``mha.`` level in their key (tt_bio/tenstorrent.py:973, 981 strip it; the Protenix / ESMFold2 remaps
    emit keys without it, tt_bio/protenix_weights.py:80-83).  Accept both: insert the level where it is missing."""
    for key in list(state_dict.keys()):
        if not key.startswith(prefix):
            continue
        m = _TRI_ATT_KEY.search(key)
        if m is not None:
            state_dict[key[:m.end(1)] + "mha." + key[m.end(1):]] = state_dict.pop(key)


def _run_layers(layers, s, z, mask, pair_mask, ws_cache: Optional[dict] = None, inplace: bool = False):
    """``inplace``: s [N, c_s] and z [N, N, C] are the caller's fp32 contiguous working tensors and are updated
    where they are (nothing is returned); otherwise [1, ...] inputs are copied and new tensors returned."""
    if not z.is_cuda:
        raise RuntimeError("B200 Pairformer: inputs must be CUDA tensors (there is no CPU path)")
    if inplace:
        if z.dim() != 3 or z.shape[0] != z.shape[1] or z.dtype != torch.float32 or not z.is_contiguous():
            raise RuntimeError("B200 Pairformer: the in-place form takes a contiguous fp32 z [N, N, C]")
        if s is not None and (s.dtype != torch.float32 or not s.is_contiguous() or s.dim() != 2):
            raise RuntimeError("B200 Pairformer: the in-place form takes a contiguous fp32 s [N, c_s]")
    elif z.dim() != 4 or z.shape[0] != 1 or z.shape[1] != z.shape[2]:
        raise RuntimeError(f"B200 Pairformer: z must be [1, N, N, C], got {tuple(z.shape)}")
    n = z.shape[-2]
    with torch.cuda.device(z.device), torch.no_grad():
        if inplace:
            zw, sw = z, s
        else:
            zw = z[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
            sw = None if s is None else s[0].to(torch.float32).clone(memory_format=torch.contiguous_format)
        pm = ops.PairMasks(_mask_u8(pair_mask, (n, n), z.device))
        tm = _mask_u8(mask, (n,), z.device) if s is not None else None
        ws = None
        if any(l.fused for l in layers):
            key = (n, z.device)
            if ws_cache is not None and key in ws_cache:
                ws = ws_cache[key]
            else:
                ws = ops.Workspace(n, z.device)
                if ws_cache is not None:
                    ws_cache.clear()
                    ws_cache[key] = ws
        side = None
        if sw is not None and len(layers) > 1 and os.environ.get("B200PF_SIDE_TRACK", "0") == "1":
            side = SideTrack(z.device)
        for layer in layers:
            layer.forward_inplace(sw, zw, tm, pm, ws, side)
        if side is not None:
            side.join()
    if inplace:
        return None
    z_out = zw.unsqueeze(0).to(z.dtype)
    s_out = None if sw is None else sw.unsqueeze(0).to(s.dtype)
    return s_out, z_out


class B200PairformerModule(nn.Module):
    """Stack of Pairformer blocks behind both of the reference's constructors.

    * CPU modules' style (tt_bio/reference.py:921-934): ``(token_s, token_z, num_blocks, num_heads=16,
      dropout=0.25, pairwise_head_width=32, pairwise_num_heads=4, post_layer_norm=False,
      activation_checkpointing=False, v2=False)``
    * device backend's style (tt_bio/tenstorrent.py:2194-2204): ``(n_blocks, tri_att_head_dim, tri_att_n_heads,
      att_head_dim, att_n_heads, transform_s, affinity=False)``; chosen when ``transform_s`` is given (sixth
      positional argument or keyword).  ``transform_s=False`` builds pair-only blocks and ``forward`` then
      takes ``s=None`` and returns ``(None, z)``.  The pair width is not part of that signature (the backend
      reads it off the weights); it is 128 unless ``token_z=`` says otherwise.  ``affinity`` only selects how the
      backend builds its masks; here every call honours the full 2-D ``pair_mask`` like the CPU modules.

    ``forward(s, z, mask=None, pair_mask=None, use_kernels=False) -> (s, z)`` in both cases; a missing
    ``pair_mask`` is the outer product of ``mask`` (all ones when that is missing too), which is what the
    backend derives from the token mask (tt_bio/tenstorrent.py:2257-2267).
    """

    def __init__(self, *args, precision: str = "bf16", **kwargs) -> None:
        super().__init__()
        if "transform_s" in kwargs or (len(args) >= 6 and isinstance(args[5], bool)):
            names = ("n_blocks", "tri_att_head_dim", "tri_att_n_heads", "att_head_dim", "att_n_heads", "transform_s", "affinity")
            if len(args) > len(names):
                raise TypeError("too many positional arguments for the backend-style constructor")
            cfg = dict(zip(names, args))
            for k in names:
                if k in kwargs:
                    cfg[k] = kwargs.pop(k)
            missing = [k for k in names[:6] if k not in cfg]
            if missing:
                raise TypeError(f"backend-style constructor: missing {missing}")
            with_s = bool(cfg["transform_s"])
            num_blocks = int(cfg["n_blocks"])
            token_z = int(kwargs.pop("token_z", 128))
            num_heads = int(cfg["att_n_heads"]) if with_s else 16
            token_s = int(kwargs.pop("token_s", num_heads * int(cfg["att_head_dim"]) if with_s else 384))
            head_width, tri_heads = int(cfg["tri_att_head_dim"]), int(cfg["tri_att_n_heads"])
            self.affinity = bool(cfg.get("affinity", False))
            dropout, post_layer_norm, v2 = 0.0, False, True
        else:
            names = ("token_s", "token_z", "num_blocks", "num_heads", "dropout", "pairwise_head_width",
                     "pairwise_num_heads", "post_layer_norm", "activation_checkpointing", "v2")
            if len(args) > len(names):
                raise TypeError("too many positional arguments")
            cfg = {"num_heads": 16, "dropout": 0.25, "pairwise_head_width": 32, "pairwise_num_heads": 4,
                   "post_layer_norm": False, "activation_checkpointing": False, "v2": False}
            cfg.update(zip(names, args))
            for k in names:
                if k in kwargs:
                    cfg[k] = kwargs.pop(k)
            missing = [k for k in names[:3] if k not in cfg]
            if missing:
                raise TypeError(f"missing constructor arguments {missing}")
            with_s, num_blocks = True, int(cfg["num_blocks"])
            token_s, token_z, num_heads = int(cfg["token_s"]), int(cfg["token_z"]), int(cfg["num_heads"])
            head_width, tri_heads = int(cfg["pairwise_head_width"]), int(cfg["pairwise_num_heads"])
            dropout, post_layer_norm, v2 = cfg["dropout"], cfg["post_layer_norm"], cfg["v2"]
            self.affinity = False
        self.token_z, self.num_blocks, self.num_heads, self.transform_s = token_z, num_blocks, num_heads, with_s
        self.layers = nn.ModuleList([
            B200PairformerLayer(token_s, token_z, num_heads, dropout, head_width, tri_heads,
                                post_layer_norm, v2, precision, with_s=with_s) for _ in range(num_blocks)])
        self._ws_cache: dict = {}
        self._register_load_state_dict_pre_hook(_accept_backend_keys)

    def reset_static_cache(self) -> None:
        self._ws_cache.clear()
        for layer in self.layers:
            layer.reset_static_cache()

    def run_inplace(self, s: Optional[torch.Tensor], z: torch.Tensor, mask: Optional[torch.Tensor] = None,
                    pair_mask: Optional[torch.Tensor] = None) -> None:
        """The stack on the caller's resident fp32 tensors s [N, c_s] and z [N, N, C], updated in place: the form a
        recycling loop uses to keep z on the device between passes (see ``B200RecyclingTrunk``)."""
        if pair_mask is None and mask is not None:
            m = mask.reshape(1, -1).to(z.device)
            pair_mask = m[:, :, None] * m[:, None, :]
        _run_layers(list(self.layers), s if self.transform_s else None, z, mask if self.transform_s else None, pair_mask,
                    self._ws_cache, inplace=True)

    def forward(self, s: Optional[torch.Tensor], z: torch.Tensor, mask: Optional[torch.Tensor] = None,
                pair_mask: Optional[torch.Tensor] = None, use_kernels: bool = False
                ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        if pair_mask is None and mask is not None:
            m = mask.reshape(1, -1).to(z.device)
            pair_mask = m[:, :, None] * m[:, None, :]
        if not self.transform_s:
            return None, _run_layers(list(self.layers), None, z, None, pair_mask, self._ws_cache)[1]
        if s is None:
            raise RuntimeError("B200PairformerModule: this stack has a single track; s must be given")
        return _run_layers(list(self.layers), s, z, mask, pair_mask, self._ws_cache)


class B200PairformerNoSeqModule(nn.Module):
    """Pair-only stack (templates, affinity, MSA pair stack): forward(z, pair_mask) -> z."""

    def __init__(self, token_z: int, num_blocks: int, dropout: float = 0.25, pairwise_head_width: int = 32,
                 pairwise_num_heads: int = 4, post_layer_norm: bool = False, activation_checkpointing: bool = False,
                 precision: str = "bf16", **kwargs) -> None:
        super().__init__()
        self.token_z, self.num_blocks = token_z, num_blocks
        self.layers = nn.ModuleList([
            B200PairformerNoSeqLayer(token_z, dropout, pairwise_head_width, pairwise_num_heads, post_layer_norm, precision)
            for _ in range(num_blocks)])
        self._ws_cache: dict = {}
        self._register_load_state_dict_pre_hook(_accept_backend_keys)

    def reset_static_cache(self) -> None:
        self._ws_cache.clear()
        for layer in self.layers:
            layer.reset_static_cache()

    def forward(self, z: torch.Tensor, pair_mask: Optional[torch.Tensor] = None, use_kernels: bool = False
                ) -> torch.Tensor:
        return _run_layers(list(self.layers), None, z, None, pair_mask, self._ws_cache)[1]
