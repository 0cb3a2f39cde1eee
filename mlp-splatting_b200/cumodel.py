"""Drop-in renderer module for the inference path of scannet/cumodel.py.

`NeuralPrimitiveSceneTileCUDA` keeps the reference class's constructor arguments, parameter
names and shapes (cumodel.py:655-743), `set_image_size`, `forward` (cumodel.py:951-1160) and the
no-grad helpers `render_feature_map`, `render_rgb_alpha_no_grad`, `render_rgb_t_no_grad`
(cumodel.py:1162-1525).  Rendering runs on the sm_100a kernels behind libmlpsp_b200.so; there is
no autograd (training is out of scope) and no CPU path.

Differences a caller can see:
  * tile_size 16 (which the reference takes for its scalar kernels) culls and orders per 16x16 tile and renders on
    8x8 tiles that inherit those lists: same candidates and order per pixel; mosaic culling stays 8x8;
  * `precision` ("fp16" default, or "fp32") selects the evaluator: fp16 matches the reference's
    tensor-core forward (scannet/cuda/rgb_wmma.cuh), fp32 its scalar forward;
  * culling, sorting and rendering are one asynchronous launch sequence followed by one status
    read-back, where the reference synchronises on `tile_prim_pairs.numel()` (cumodel.py:1055) and
    again inside its validator (np_tile_kernels.cu:4576).
"""
from __future__ import annotations

import os

import torch
from torch import nn

from . import _lib as L
from .engine import FrameRenderer, PackedScene


def _tile_ext_build_config(tile_size=None):
    """The reference's extension build configuration (cumodel.py:96-130) as run-time configuration.

    The reference compiles one extension per combination of these environment variables (-D flags); this
    library's kernels take the same quantities as arguments of a call, so the variables select arguments:
      MLPSP_TILE_CANDIDATE_CAPACITY  768 or 1536 (default)  -> FrameRenderer(tile_capacity=...), and with it the
                                                               "tile candidate capacity N exceeded" error
      MLPSP_TRAINING_BACKEND=csr with MLPSP_CSR_MAX_HITS     128 (default), 256 or 512 -> max_hits of the record export
      MLPSP_NVCC_MAXRREGCOUNT        accepted and ignored: the register budgets belong to this library's own kernels
    Same checks and error texts as the reference."""
    tile_candidates = int(os.environ.get("MLPSP_TILE_CANDIDATE_CAPACITY", "1536"))
    if tile_candidates not in {768, 1536}:
        raise ValueError("MLPSP_TILE_CANDIDATE_CAPACITY must be 768 or 1536")
    max_hits = None
    if os.environ.get("MLPSP_TRAINING_BACKEND", "legacy") == "csr":
        max_hits = int(os.environ.get("MLPSP_CSR_MAX_HITS", "128"))
        if max_hits not in {128, 256, 512}:
            raise ValueError("MLPSP_CSR_MAX_HITS must be 128, 256 or 512; overflow is an error")
    return {"tile_candidate_capacity": tile_candidates, "csr_max_hits": max_hits,
            "tile_size": 8 if tile_size is None else int(tile_size)}


class IntegratedPositionalEncoding(nn.Module):
    """Frequencies 2^k * pi and attenuation exp(-0.5 f^2 sigma^2) (cumodel.py:132-155)."""

    def __init__(self, in_dim=6, num_frequencies=10, sigma=0.01):
        super().__init__()
        self.in_dim, self.num_frequencies, self.sigma2 = in_dim, num_frequencies, sigma ** 2
        self.register_buffer("freq_bands", 2.0 ** torch.linspace(0.0, num_frequencies - 1, num_frequencies) * torch.pi)
        self.register_buffer("runtime_frequency_weights", torch.ones(num_frequencies), persistent=False)

    def set_runtime_frequency_weights(self, weights):
        with torch.no_grad():
            self.runtime_frequency_weights.copy_(weights.to(self.runtime_frequency_weights))

    def attenuation(self):
        return torch.exp(-0.5 * (self.freq_bands ** 2) * self.sigma2) * self.runtime_frequency_weights

    @property
    def out_dim(self):
        return self.in_dim * self.num_frequencies * 2


class FourierFeatureEncoding(nn.Module):
    """Frequencies 2^k, unit attenuation (cumodel.py:158-180)."""

    def __init__(self, in_dim=6, num_frequencies=10):
        super().__init__()
        self.in_dim, self.num_frequencies = in_dim, num_frequencies
        self.register_buffer("freq_bands", 2.0 ** torch.linspace(0.0, num_frequencies - 1, num_frequencies))
        self.register_buffer("runtime_frequency_weights", torch.ones(num_frequencies), persistent=False)

    def set_runtime_frequency_weights(self, weights):
        with torch.no_grad():
            self.runtime_frequency_weights.copy_(weights.to(self.runtime_frequency_weights))

    def attenuation(self):
        return self.runtime_frequency_weights.clone()

    @property
    def out_dim(self):
        return self.in_dim * self.num_frequencies * 2


class NeuralPrimitiveSceneTileCUDA(nn.Module):
    """Tile-based MLP splatting renderer (inference), same call surface as the reference class."""

    requires_full_image = True

    def __init__(self, num_primitives=1024, hidden_dim=32, pe_frequencies=6, initial_positions=None,
                 use_integrated_pe=True, pe_sigma: float = 0.01, min_points: int = 10, tile_size: int = 8,
                 feature_dim_low: int = 0, feature_slots: int = 4, feature_gating_beta: float = 1.5,
                 feature_gating_temp: float = 2.0, precision: str = "fp16", wide_hidden: bool = False):
        """The reference's arguments (scannet/cumodel.py:664-685) plus precision and wide_hidden.  wide_hidden=True
        lifts the reference's hidden_dim <= 32 limit to the 64 this library's evaluators take (the tensor-core
        evaluator at 32 and 64, the FP32 one at any width up to 64); nothing of the reference computes such a
        network, so it is checked against the CPU restatement only."""
        super().__init__()
        if int(hidden_dim) > 32 and not wide_hidden:
            raise ValueError("NeuralPrimitiveSceneTileCUDA currently supports hidden_dim <= 32 "
                             "(kernel scratch-cap tuning in backward/full path).")
        if int(hidden_dim) > 64:
            raise ValueError("hidden_dim beyond 64 is not supported")
        if float(pe_sigma) <= 0.0:
            raise ValueError("pe_sigma must be > 0.")
        if int(tile_size) <= 0:
            raise ValueError("tile_size must be a positive integer.")
        if int(tile_size) not in (8, 16):
            raise ValueError("NeuralPrimitiveSceneTileCUDA supports tile_size in {8, 16}.")
        if initial_positions is not None:
            raise ValueError("octree initialisation from a point cloud belongs to training and is not part of this build")
        if precision not in ("fp16", "bf16", "fp32"):
            raise ValueError("precision must be 'fp16', 'bf16' or 'fp32'")
        self.num_primitives = int(num_primitives)
        self.hidden_dim, self.pe_frequencies = int(hidden_dim), int(pe_frequencies)
        self.use_integrated_pe, self.pe_sigma = bool(use_integrated_pe), float(pe_sigma)
        self.image_size = None
        self.tile_size = int(tile_size)
        self.tile_order_mode_override = None
        self.feature_dim_low = int(max(0, feature_dim_low))
        self.feature_slots = int(max(1, feature_slots))
        self.feature_gating_beta, self.feature_gating_temp = float(feature_gating_beta), float(feature_gating_temp)
        if self.feature_dim_low > 0 and self.feature_slots not in (4, 5):
            raise ValueError("feature_slots must be 4 (canonical) or 5 (legacy) when features are enabled.")
        if self.feature_gating_beta <= 0.0:
            raise ValueError("feature_gating_beta must be > 0.")
        if self.feature_gating_temp <= 0.0:
            raise ValueError("feature_gating_temp must be > 0.")
        self.precision = precision
        n, H = self.num_primitives, self.hidden_dim
        self.positions = nn.Parameter(torch.rand(n, 3) * 2 - 1)
        self.log_scales = nn.Parameter(torch.log(torch.ones(n) * 0.1).unsqueeze(-1).repeat(1, 3))
        self.quats = nn.Parameter(torch.tensor([1.0, 0.0, 0.0, 0.0]).view(1, 4).repeat(n, 1))
        self.encoder = (IntegratedPositionalEncoding(6, pe_frequencies, self.pe_sigma) if self.use_integrated_pe
                        else FourierFeatureEncoding(6, pe_frequencies))
        IN = self.encoder.out_dim
        self.W1 = nn.Parameter(torch.randn(n, H, IN) * 0.01)
        self.b1 = nn.Parameter(torch.zeros(n, H))
        self.W2 = nn.Parameter(torch.randn(n, H, H) * 0.01)
        self.b2 = nn.Parameter(torch.zeros(n, H))
        self.W3 = nn.Parameter(torch.randn(n, 4, H) * 0.01)
        self.b3 = nn.Parameter(torch.zeros(n, 4))
        if self.feature_dim_low > 0:
            if self.feature_slots == 5:
                fi = torch.zeros(n, 5, self.feature_dim_low)
                fi[:, 0, :].normal_(mean=0.0, std=0.01)
            else:
                fi = torch.randn(n, self.feature_slots, self.feature_dim_low) * 0.01
            self.feat_attr = nn.Parameter(fi)
        else:
            self.feat_attr = None
        for name, dt in (("stat_sum_w", torch.float32), ("stat_max_w", torch.float32), ("stat_hits", torch.int32),
                         ("stat_contrib_count", torch.int32), ("stat_sum_werr", torch.float32)):
            self.register_buffer(name, torch.zeros(n, dtype=dt))
        self._packed = None
        self._packed_key = None
        self._renderers = {}

    # ------------------------------------------------------------------ reference surface ----
    def set_image_size(self, W: int, H: int):
        self.image_size = (int(W), int(H))

    def _activate_cuda_device(self) -> torch.device:
        device = self.positions.device
        if device.type != "cuda":
            raise RuntimeError("NeuralPrimitiveSceneTileCUDA must be moved to a CUDA device before rendering.")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(device.index)
        return device

    def _resolve_tile_order_mode(self) -> str:
        mode = self.tile_order_mode_override
        if mode is None or str(mode).strip() == "":
            mode = os.environ.get("MLPSP_TILE_ORDER", "tilecenter")
        mode = {"tile_center": "tilecenter", "tile-center": "tilecenter"}.get(str(mode).strip().lower(),
                                                                              str(mode).strip().lower())
        if mode not in {"tilecenter", "per_pixel"}:
            raise ValueError(f"Unknown tile order mode: {mode}")
        return mode

    # --------------------------------------------------------------------------- internals ----
    def _params(self):
        ps = [self.positions, self.log_scales, self.quats, self.W1, self.b1, self.W2, self.b2, self.W3, self.b3]
        if self.feat_attr is not None:
            ps.append(self.feat_attr)
        return ps

    def packed_scene(self) -> PackedScene:
        """Packed parameters on the module's device, rebuilt when a parameter changed in place."""
        device = self._activate_cuda_device()
        w = self.encoder.runtime_frequency_weights
        key = (str(device), self.precision) + tuple((p.data_ptr(), p._version) for p in self._params()) + \
              (w.data_ptr(), w._version)
        if self._packed is None or self._packed_key != key:
            with torch.no_grad():
                freq = self.encoder.freq_bands.to(device=device, dtype=torch.float32)
                att = self.encoder.attenuation().to(device=device, dtype=torch.float32)
                self._packed = PackedScene(
                    self.positions.detach(), self.log_scales.detach(), self.quats.detach(), self.W1.detach(),
                    self.b1.detach(), self.W2.detach(), self.b2.detach(), self.W3.detach(), self.b3.detach(), freq, att,
                    feat_attr=None if self.feat_attr is None else self.feat_attr.detach(),
                    gate_beta=self.feature_gating_beta, gate_tau=self.feature_gating_temp, device=device,
                    pack_f16=(self.precision == "fp16"), pack_bf16=(self.precision == "bf16"))
            self._packed_key = key
        return self._packed

    def _renderer(self, device) -> FrameRenderer:
        W, H = self.image_size
        capacity = _tile_ext_build_config(self.tile_size)["tile_candidate_capacity"]
        key = (str(device), W, H, capacity)
        if key not in self._renderers:
            self._renderers[key] = FrameRenderer(W, H, device=device, tile_capacity=capacity)
        return self._renderers[key]

    def _render(self, ray_o, ray_d, score_threshold, bg_color, view_matrix, proj_matrix, culled_prim_indices,
                tile_offsets, want_depth, path_name, want_feat=False, sort_key=0, stats=None):
        if self.image_size is None:
            raise ValueError("image_size must be set on NeuralPrimitiveSceneTileCUDA before calling forward.")
        W, H = self.image_size
        if ray_o.shape[0] != W * H:
            raise AssertionError("Tile renderer requires full-frame rays (B == W*H)")
        device = self._activate_cuda_device()
        if self._resolve_tile_order_mode() == "per_pixel":
            # render_tiles_forward (np_tile_kernels.cu:714-926): every pixel blends its own hits in its own order
            if want_depth or stats is not None:
                raise ValueError("per_pixel ordering renders rgb, alpha and the feature map only here; use "
                                 "MLPSP_TILE_ORDER=tilecenter for depth and contribution statistics")
            sort_key = L.ORDER_PER_PIXEL
        ts = int(self.tile_size)
        if ts == 16 and (sort_key == L.ORDER_PER_PIXEL or getattr(self, "camera_mode", "legacy-centered") == "colmap-native"):
            raise ValueError("tile_size = 16 renders the tile-centre order with screen-space or external culling only")
        T = ((W + ts - 1) // ts) * ((H + ts - 1) // ts)
        lists = None
        if getattr(self, "camera_mode", "legacy-centered") == "colmap-native":
            if (culled_prim_indices is not None) or (tile_offsets is not None):
                raise ValueError("Native camera culling must be derived from the actual rays")
            from .camera import ray_cone_candidates
            culled_prim_indices, tile_offsets = ray_cone_candidates(
                ray_o.detach().float().contiguous(), ray_d.detach().float().contiguous(), self.positions.detach(),
                self.log_scales.detach(), W, H, 8, float(score_threshold), scene=self.packed_scene(),
                renderer=self._renderer(device))
        if (culled_prim_indices is not None) or (tile_offsets is not None):
            if culled_prim_indices is None or tile_offsets is None:
                raise ValueError("Both culled_prim_indices and tile_offsets must be provided together.")
            cp = culled_prim_indices.to(device=device, dtype=torch.int32).contiguous()
            to = tile_offsets.to(device=device, dtype=torch.int32).contiguous()
            if to.numel() != T + 1:
                raise ValueError(f"tile_offsets length mismatch: got {to.numel()}, expected {T + 1}")
            lists = (cp, to)
        elif view_matrix is None or proj_matrix is None:
            raise ValueError("Tile renderer requires view_matrix/proj_matrix unless external culling is provided.")
        scene = self.packed_scene()
        r = self._renderer(device)
        bg = None
        if bg_color is not None:
            bg = torch.as_tensor(bg_color, dtype=torch.float32).detach().cpu().reshape(-1)
            bg = bg.repeat(3) if bg.numel() == 1 else bg
            bg = bg.numpy()
        view = None if lists is not None else view_matrix.detach().float().cpu().numpy()
        proj = None if lists is not None else proj_matrix.detach().float().cpu().numpy()
        prec = L.PRECISION_F32
        if self.precision == "fp16" and scene.has_f16:
            prec = L.PRECISION_F16
        elif self.precision == "bf16" and scene.has_bf16:
            prec = L.PRECISION_BF16
        render = r.render_tile16 if ts == 16 else r.render      # 16x16: culling and order per 16x16 tile, as the reference
        rgb, alpha = render(scene, ray_o.detach().float().contiguous(), ray_d.detach().float().contiguous(),
                            float(score_threshold), view=view, proj=proj, precision=prec, bg=bg,
                            want_depth=want_depth, tile_lists=lists, path_name=path_name, want_feat=want_feat,
                            sort_key=sort_key, prim_stats=stats)
        return r, rgb, alpha

    @torch.no_grad()
    def build_tilecenter_culling_from_tile_views(self, tile_view_ids, view_matrices, proj_matrix,
                                                 score_threshold: float = 1e-3, tile_size=None):
        """Tile->primitive lists for a mosaic frame (per-tile view assignment), cumodel.py:838-949.
        Returns (culled_prim_indices int32 [M], tile_offsets int32 [T+1]), ascending id inside a tile."""
        if getattr(self, "camera_mode", "legacy-centered") == "colmap-native":
            return None, None
        if self.image_size is None:
            raise ValueError("image_size must be set before building tile culling.")
        device = self._activate_cuda_device()
        ts = int(self.tile_size if tile_size is None else tile_size)
        if ts <= 0:
            raise ValueError("tile_size must be a positive integer.")
        if ts != 8:
            raise ValueError("this build renders 8x8 tiles only")
        W, H = self.image_size
        T = ((W + 7) // 8) * ((H + 7) // 8)
        tv = torch.as_tensor(tile_view_ids).reshape(-1)
        if tv.numel() != T:
            raise ValueError(f"tile_view_ids length mismatch: got {tv.numel()}, expected {T}")
        vm = torch.as_tensor(view_matrices)
        if vm.ndim != 3 or tuple(vm.shape[1:]) != (4, 4):
            raise ValueError("view_matrices must have shape (K,4,4)")
        if int(vm.shape[0]) <= 0:
            raise ValueError("view_matrices must contain at least one view")
        prims, offs = self._renderer(device).bin_mosaic(self.packed_scene(), tv, vm.detach().float().cpu().numpy(),
                                                        torch.as_tensor(proj_matrix).detach().float().cpu().numpy(),
                                                        float(score_threshold))
        return prims.clone(), offs.clone()

    # ----------------------------------------------------------------------------- public ----
    @torch.no_grad()
    def forward(self, ray_o, ray_d, score_threshold=1e-3, bg_color=None, view_matrix=None, proj_matrix=None,
                culled_prim_indices=None, tile_offsets=None, return_feature: bool = False, feature_target=None):
        """Same arguments as the reference forward (cumodel.py:951-963); returns rgb [W*H,3]
        (a fresh tensor), or (rgb, feat) when return_feature is set and features exist."""
        if feature_target is not None:
            raise ValueError("CSR feature training is outside the inference render path")
        if return_feature and self.feat_attr is None:
            raise RuntimeError("return_feature=True requested but feat_attr is not initialized.")
        if return_feature:
            r, rgb, _alpha = self._render(ray_o, ray_d, score_threshold, bg_color, view_matrix, proj_matrix,
                                          culled_prim_indices, tile_offsets, False,
                                          "render_tiles_forward_tilecenter_with_feat", want_feat=True)
            return rgb.clone(), r.feat.clone()
        _r, rgb, _alpha = self._render(ray_o, ray_d, score_threshold, bg_color, view_matrix, proj_matrix,
                                       culled_prim_indices, tile_offsets, False, "render_tiles_forward_tilecenter")
        return rgb.clone()

    @torch.no_grad()
    def render_rgb_alpha_no_grad(self, ray_o, ray_d, score_threshold=1e-3, bg_color=None, view_matrix=None,
                                 proj_matrix=None, collect_w_stats=False, gt_rgb=None, culled_prim_indices=None,
                                 tile_offsets=None):
        """(rgb [B,3], alpha [B,1]) as cumodel.py:1196-1383.  collect_w_stats accumulates the per-primitive
        contribution statistics w = T * alpha into stat_sum_w / stat_max_w / stat_hits / stat_sum_werr /
        stat_contrib_count, which needs the ground-truth image."""
        if getattr(self, "camera_mode", "legacy-centered") == "colmap-native":
            raise NotImplementedError("Native camera statistics rendering is not implemented; use forward for RGB/features")
        stats = None
        if collect_w_stats:
            if self.image_size is None:
                raise ValueError("image_size must be set on NeuralPrimitiveSceneTileCUDA before calling render_rgb_alpha_no_grad.")
            B = self.image_size[0] * self.image_size[1]
            if gt_rgb is None:
                raise ValueError("collect_w_stats=True requires gt_rgb (shape=(B,3), B=W*H) to compute pixel_error inside the CUDA kernel.")
            if gt_rgb.dim() != 2 or gt_rgb.shape[0] != B or gt_rgb.shape[1] != 3:
                raise ValueError(f"gt_rgb must have shape (B,3) with B=W*H={B}, got {tuple(gt_rgb.shape)}")
            device = self._activate_cuda_device()
            gt = gt_rgb.to(device=device, dtype=torch.float32).contiguous()
            for name, dt in (("stat_sum_w", torch.float32), ("stat_max_w", torch.float32), ("stat_hits", torch.int32),
                             ("stat_sum_werr", torch.float32), ("stat_contrib_count", torch.int32)):
                buf = getattr(self, name, None)
                if buf is None or buf.numel() != self.num_primitives or buf.device != device:
                    setattr(self, name, torch.zeros(self.num_primitives, dtype=dt, device=device))
            stats = (gt, self.stat_sum_w, self.stat_max_w, self.stat_hits, self.stat_sum_werr, self.stat_contrib_count)
        # the reference's statistics kernel orders a tile by the Euclidean depth of the centres along the
        # tile-centre ray (np_tile_kernels.cu:2248-2256), its plain forward by t*: both are kept
        _r, rgb, alpha = self._render(ray_o, ray_d, score_threshold, bg_color, view_matrix, proj_matrix,
                                      culled_prim_indices, tile_offsets, False, "render_tiles_forward_tilecenter",
                                      stats=stats, sort_key=1 if stats is not None else 0)
        return rgb.clone(), alpha.clone()

    @torch.no_grad()
    def reset_w_stats(self):
        """Zero the per-primitive contribution statistics (cumodel.py:764-774)."""
        dev = self.positions.device
        n = self.positions.shape[0]
        self.stat_sum_w = torch.zeros(n, device=dev, dtype=torch.float32)
        self.stat_hits = torch.zeros(n, device=dev, dtype=torch.int32)
        self.stat_max_w = torch.zeros(n, device=dev, dtype=torch.float32)
        self.stat_sum_werr = torch.zeros(n, device=dev, dtype=torch.float32)
        self.stat_contrib_count = torch.zeros(n, device=dev, dtype=torch.int32)

    @torch.no_grad()
    def render_rgb_t_no_grad(self, ray_o, ray_d, score_threshold=1e-3, bg_color=None, view_matrix=None,
                             proj_matrix=None, culled_prim_indices=None, tile_offsets=None):
        """(rgb, expected depth t [B,1], alpha) as cumodel.py:1385-1525.  The reference's expected-depth
        kernel orders a tile by Euclidean depth along the tile-centre ray (np_tile_kernels.cu:5538-5543),
        not by t*, so this call does too."""
        r, rgb, alpha = self._render(ray_o, ray_d, score_threshold, bg_color, view_matrix, proj_matrix,
                                     culled_prim_indices, tile_offsets, True, "render_tiles_forward_tilecenter_with_t",
                                     sort_key=1)
        return rgb.clone(), r.depth_t.clone(), alpha.clone()

    @torch.no_grad()
    def render_feature_map(self, ray_o, ray_d, score_threshold=1e-3, view_matrix=None, proj_matrix=None,
                           culled_prim_indices=None, tile_offsets=None):
        if self.feat_attr is None:
            raise RuntimeError("Feature rendering requested but feature_dim_low == 0.")
        if self.image_size is None:
            raise ValueError("image_size must be set before calling render_feature_map.")
        W, H = self.image_size
        if ray_o.shape[0] != W * H:
            raise ValueError("render_feature_map requires full-frame rays (B == W*H).")
        _rgb, feat = self.forward(ray_o=ray_o, ray_d=ray_d, score_threshold=score_threshold, bg_color=None,
                                  view_matrix=view_matrix, proj_matrix=proj_matrix,
                                  culled_prim_indices=culled_prim_indices, tile_offsets=tile_offsets,
                                  return_feature=True)
        return feat


@torch.no_grad()
def render_tiles_training_records(tensors, width, height, tile, threshold, beta, temperature, precision="float32",
                                  max_hits=None):
    """Forward record list with the argument list of the reference's extension entry points
    render_tiles_training_records / render_tiles_training_records_wmma (np_tile_kernels.cu:6994,
    training_wmma.cuh:270): `tensors` = [rays_o, rays_d (unit), positions, log_scales, quats (unit),
    culled_prim_indices, tile_offsets, freq, att, W1, b1, W2, b2, W3, b3] (two trailing adjoint
    placeholders are accepted and ignored).  Returns [rgb, alpha, ids, x6, raw, masks, gates, offsets].
    precision "float32" selects the scalar evaluator, "float16" the tensor-core one.  max_hits (records per pixel;
    more is an error) defaults to MLPSP_CSR_MAX_HITS when MLPSP_TRAINING_BACKEND=csr is set, else to 512."""
    cfg = _tile_ext_build_config(tile)
    if max_hits is None:
        max_hits = cfg["csr_max_hits"] or 512
    if len(tensors) not in (15, 17):
        raise ValueError("expected the 15 scene tensors (optionally followed by two adjoint placeholders)")
    if int(tile) != 8:
        raise ValueError("Training WMMA requires tile8")
    if precision not in ("float32", "float16"):
        raise ValueError("precision must be float32 or float16")
    ro, rd, pos, ls, q, culled, offs, freq, att, W1, b1, W2, b2, W3, b3 = tensors[:15]
    dev = ro.device
    scene = PackedScene(pos, ls, q, W1, b1, W2, b2, W3, b3, freq, att, gate_beta=float(beta), gate_tau=float(temperature),
                        device=dev, pack_f16=(precision == "float16"))
    r = FrameRenderer(int(width), int(height), device=dev, max_pairs=max(int(culled.numel()), 1),
                      tile_capacity=cfg["tile_candidate_capacity"])
    prec = L.PRECISION_F16 if (precision == "float16" and scene.has_f16) else L.PRECISION_F32
    return r.render_records(scene, ro.contiguous().float(), rd.contiguous().float(), float(threshold), max_hits=max_hits,
                            precision=prec, tile_lists=(culled, offs), rays_normalized=True,
                            path_name="render_tiles_training_records")
