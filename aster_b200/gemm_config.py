"""GEMM operator surface: problem, mapping, validated instance and label grammar.

Host-side mirror of the reference's ``contrib/kittens/gemm_config.py`` so that configs, sweeps
and stored labels written for the reference keep working:

* :class:`GemmSpec` -- the problem ``C[M,N] += A[M,K] . B[N,K]`` with packed row-major byte
  layouts (gemm_config.py:90-205).
* :class:`GemmMappingSpec` -- workgroup grid, wave grid, tiles per wave, pipeline strategy,
  operand path and the scheduling knobs, with the reference's resource estimators
  (gemm_config.py:213-446).
* :class:`WeakScaledMappedGemmInstance` -- a (spec, mapping) pair that satisfies the weak-scale
  identity ``M == wg_m * twg_m * mfma_m`` and serialises to / parses from the label grammar
  (gemm_config.py:509-719).

What the fields mean on B200 is decided by :class:`B200GemmInstance` at the bottom: the
16x16 MFMA tile is only the accounting unit, the workgroup tile selects the CTA tile width,
the pipeline strategy's depth selects the shared-memory ring depth, and the AMD scheduling
knobs are carried in the label but do not change the kernel.
"""

from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from enum import Enum
from typing import Optional

from .kittens_helpers import PIPELINE_STRATEGIES


class LoadType(Enum):
    FLAT = "flat"
    BUFFER = "buffer"


class OperandPath(Enum):
    LDS = "lds"  # A and B staged in shared memory from row-major global tensors
    DIRECT_B = "direct_b"  # B arrives pre-arranged and skips the layout-transforming load
    DIRECT_AB = "direct_ab"


class Operand(Enum):
    A = "a"
    B = "b"
    C = "c"


A, B, C = Operand.A, Operand.B, Operand.C
DIM_M, DIM_N, DIM_K = 0, 1, 2

_MFMA_SHAPE_FOR_MCPU = {"gfx942": [16, 16, 16], "gfx950": [16, 16, 32], "sm_100a": [16, 16, 16]}


def mfma_shape_for_mcpu(mcpu: str) -> list[int]:
    """Accounting tile ``[m, n, k]`` per target (gemm_config.py:74-82)."""
    return list(_MFMA_SHAPE_FOR_MCPU.get(mcpu, [16, 16, 16]))


class Layout:
    """Flat strided layout: the slice of ``aster.layout.Layout`` value semantics the operator
    surface needs (python/aster/layout/algebra.py:53-141): sizes, strides, ``size()``,
    ``is_flat``, evaluation of a linear index, equality."""

    __slots__ = ("sizes", "strides")

    def __init__(self, sizes, strides=None) -> None:
        self.sizes = sizes
        if strides is None:
            # compact, first mode fastest -- the default of the reference class
            if isinstance(sizes, int):
                strides = 1
            else:
                acc, out = 1, []
                for s in sizes:
                    out.append(acc)
                    acc *= s
                strides = tuple(out)
        self.strides = strides

    @property
    def is_flat(self) -> bool:
        return isinstance(self.sizes, int) or all(isinstance(s, int) for s in self.sizes)

    def size(self) -> int:
        return self.sizes if isinstance(self.sizes, int) else math.prod(self.sizes)

    def __len__(self) -> int:
        return len(self.sizes) if isinstance(self.sizes, tuple) else 1

    def __call__(self, idx: int) -> int:
        if isinstance(self.sizes, int):
            return idx * self.strides
        off = 0
        for size, stride in zip(self.sizes, self.strides):
            off += (idx % size) * stride
            idx //= size
        return off

    def __eq__(self, other) -> bool:
        return isinstance(other, Layout) and self.sizes == other.sizes and self.strides == other.strides

    def __repr__(self) -> str:
        return f"Layout(sizes={self.sizes},strides={self.strides})"


class OperandLayout:
    """Per-operand geometry (gemm_config.py:454-501)."""

    def __init__(self, memory_layout: Layout, logical_dims: list[int], elt_bytes: int, mfma_shape: list[int]):
        assert memory_layout.is_flat, f"OperandLayout requires flat memory_layout, got {memory_layout!r}"
        self.memory_layout = memory_layout
        self.logical_dims = logical_dims
        self.elt_bytes = elt_bytes
        self.mfma_shape = mfma_shape

    @property
    def rank(self) -> int:
        return len(self.memory_layout)

    @property
    def shape(self) -> tuple[int, ...]:
        s = self.memory_layout.sizes
        return s if isinstance(s, tuple) else (s,)

    @property
    def strides(self) -> tuple[int, ...]:
        s = self.memory_layout.strides
        return s if isinstance(s, tuple) else (s,)

    @property
    def num_elements(self) -> int:
        return self.memory_layout.size()


@dataclass
class GemmSpec:
    """``C[dm, dn] += A[dm, dk] * B[dn, dk]`` (gemm_config.py:90-205)."""

    layout_a: Layout
    layout_b: Layout
    layout_c: Layout
    logical_dims_a: list[int] = field(default_factory=lambda: [DIM_M, DIM_K])
    logical_dims_b: list[int] = field(default_factory=lambda: [DIM_N, DIM_K])
    logical_dims_c: list[int] = field(default_factory=lambda: [DIM_M, DIM_N])
    mfma_shape: list[int] = field(default_factory=lambda: [16, 16, 16])
    elt_bytes_a: int = 2
    elt_bytes_b: int = 2
    elt_bytes_c: int = 4

    def __post_init__(self):
        self._operand_layouts = {
            Operand.A: OperandLayout(self.layout_a, self.logical_dims_a, self.elt_bytes_a, self.mfma_shape),
            Operand.B: OperandLayout(self.layout_b, self.logical_dims_b, self.elt_bytes_b, self.mfma_shape),
            Operand.C: OperandLayout(self.layout_c, self.logical_dims_c, self.elt_bytes_c, self.mfma_shape),
        }

    def operand_layout(self, operand: Operand) -> OperandLayout:
        return self._operand_layouts[operand]

    @classmethod
    def from_sizes(cls, M: int, N: int, K: int, *, elt_bytes_a: int = 2, elt_bytes_b: int = 2, elt_bytes_c: int = 4,
                   logical_dims_a=None, logical_dims_b=None, logical_dims_c=None, **kwargs) -> "GemmSpec":
        """Packed row-major byte layouts from problem sizes (gemm_config.py:136-179)."""
        extent = {DIM_M: M, DIM_N: N, DIM_K: K}
        dims = {
            "a": (logical_dims_a or [DIM_M, DIM_K], elt_bytes_a),
            "b": (logical_dims_b or [DIM_N, DIM_K], elt_bytes_b),
            "c": (logical_dims_c or [DIM_M, DIM_N], elt_bytes_c),
        }

        def packed(which: str) -> Layout:
            order, eb = dims[which]
            sizes = tuple(extent[d] for d in order)
            strides, pitch = [0] * len(sizes), eb
            for i in range(len(sizes) - 1, -1, -1):
                strides[i] = pitch
                pitch *= sizes[i]
            return Layout(sizes, tuple(strides))

        return cls(
            layout_a=packed("a"), layout_b=packed("b"), layout_c=packed("c"),
            logical_dims_a=dims["a"][0], logical_dims_b=dims["b"][0], logical_dims_c=dims["c"][0],
            elt_bytes_a=elt_bytes_a, elt_bytes_b=elt_bytes_b, elt_bytes_c=elt_bytes_c, **kwargs,
        )

    def _dim_from_operand(self, operand: Operand, dim: int) -> int:
        ol = self.operand_layout(operand)
        return ol.shape[ol.logical_dims.index(dim)]

    @property
    def gemm_size(self) -> list[int]:
        return [
            self._dim_from_operand(Operand.A, DIM_M),
            self._dim_from_operand(Operand.B, DIM_N),
            self._dim_from_operand(Operand.A, DIM_K),
        ]

    def operand_shape(self, operand: Operand) -> tuple[int, ...]:
        return self.operand_layout(operand).shape

    @property
    def total_flops(self) -> int:
        m, n, k = self.gemm_size
        return 2 * m * n * k


@dataclass
class GemmMappingSpec:
    """How the problem is laid over the GPU hierarchy (gemm_config.py:213-446)."""

    num_workgroups_per_kernel: list[int]
    num_waves_per_workgroup: list[int]
    num_tiles_per_wave: list[int]
    tile_mult: list[int] = field(default_factory=lambda: [1, 1, 2])
    pipeline_strategy: int = 1
    load_type: LoadType = LoadType.FLAT
    operand_path: OperandPath = OperandPath.LDS
    # Scheduling knobs of the reference's compiler; carried for label fidelity, no effect here.
    lcm_unroll: bool = True
    unroll_factor_multiplier: int = 1
    prologue_peeling: int = 0
    epilogue_peeling: bool = True
    ll_sched: int = 0
    hoist_wait: bool = False
    set_mfma_priority: bool = False
    rotate_compute_stage: bool = False
    use_conservative_barriers: bool = False
    global_load_bytes: int = 16
    ds_write_bytes: int = 8
    ds_read_bytes: int = 8
    mcpu: str = "sm_100a"
    num_wg_per_cu: int = 1
    wave_size: int = 64

    VGPRS_PER_LOAD = 4
    AGPRS_PER_MFMA_RESULT = 4

    def _pipeline_stage_dict(self) -> dict[str, int]:
        return PIPELINE_STRATEGIES[self.pipeline_strategy]

    @property
    def rotate_stage(self) -> Optional[int]:
        return self._pipeline_stage_dict()["COMPUTE"] if self.rotate_compute_stage else None

    @property
    def isa(self) -> str:
        return {"gfx942": "cdna3", "gfx950": "cdna4", "sm_100a": "blackwell"}.get(self.mcpu, "cdna3")

    def tile_elements(self, mfma_shape: list[int]) -> list[int]:
        return [s * m for s, m in zip(mfma_shape, self.tile_mult)]

    @staticmethod
    def default_tile_elements(mfma_shape: list[int], tile_mult: Optional[list[int]] = None) -> list[int]:
        return [s * m for s, m in zip(mfma_shape, tile_mult or [1, 1, 2])]

    @property
    def num_tiles_per_workgroup(self) -> list[int]:
        return [t * w for t, w in zip(self.num_tiles_per_wave, self.num_waves_per_workgroup)]

    @property
    def num_workgroups(self) -> int:
        return math.prod(self.num_workgroups_per_kernel)

    @property
    def num_waves(self) -> int:
        return math.prod(self.num_waves_per_workgroup)

    @property
    def num_threads(self) -> int:
        return self.num_waves * self.wave_size

    @property
    def direct_b(self) -> bool:
        return self.operand_path in (OperandPath.DIRECT_B, OperandPath.DIRECT_AB)

    @property
    def direct_a(self) -> bool:
        return self.operand_path == OperandPath.DIRECT_AB

    @property
    def use_buffer(self) -> bool:
        return self.load_type == LoadType.BUFFER

    @property
    def pipeline_depth(self) -> int:
        """Software-pipeline depth ``max(stage) + 1`` (kittens_helpers.py:161-169)."""
        return max(self._pipeline_stage_dict().values()) + 1

    # --- the reference's register / LDS accounting, kept so sweep filters and stored
    # --- expectations written against it still evaluate (gemm_config.py:358-446)
    def estimated_agprs(self) -> int:
        mt, nt, _ = self.num_tiles_per_wave
        return mt * nt * self.AGPRS_PER_MFMA_RESULT

    def _operand_vgprs(self, stages: dict[str, int], prefix: str, coop_tiles: int) -> int:
        mt, nt, kt = self.num_tiles_per_wave
        per_load = self.VGPRS_PER_LOAD
        tiles = mt * kt if prefix == "A" else kt * nt
        first, compute = stages[f"{prefix}_LOAD"], stages["COMPUTE"]
        bypass = self.direct_b if prefix == "B" else self.direct_a
        if bypass:
            return tiles * (compute - first + 1) * per_load
        extra = max(0, compute - 2)
        staged = coop_tiles * (stages[f"{prefix}_LDS_WRITE"] - first + 1) * per_load
        fragments = tiles * (compute - stages[f"{prefix}_LDS_READ"] + 1 + extra) * per_load
        return staged + fragments

    def _coop_tiles_per_wave(self) -> tuple[int, int]:
        twg, waves, kt = self.num_tiles_per_workgroup, self.num_waves, self.num_tiles_per_wave[DIM_K]

        def share(num_tiles: int) -> int:
            along_s = min(num_tiles, waves)
            along_k = max(1, waves // along_s)
            return math.ceil(num_tiles / along_s) * math.ceil(kt / along_k)

        return share(twg[DIM_M]), share(twg[DIM_N])

    def estimated_vgprs(self) -> int:
        stages = self._pipeline_stage_dict()
        coop_a, coop_b = self._coop_tiles_per_wave()
        return self._operand_vgprs(stages, "A", coop_a) + self._operand_vgprs(stages, "B", coop_b) + 10

    def lds_bytes(self, tile_bytes: int = 1024, **_overrides) -> int:
        kt = self.num_tiles_per_wave[DIM_K]
        s = self._pipeline_stage_dict()
        alloc = s["A_LOAD"] if self.direct_b else min(s["A_LOAD"], s["B_LOAD"])
        twg = self.num_tiles_per_workgroup
        total = max(1, s["A_LDS_READ"] - alloc + 1) * twg[DIM_M] * kt * tile_bytes
        if not self.direct_b:
            total += max(1, s["B_LDS_READ"] - alloc + 1) * kt * twg[DIM_N] * tile_bytes
        return total

    def simd_occupancy(self) -> int:
        return self.num_wg_per_cu * math.ceil(self.num_waves / 4)


_LABEL_RE = re.compile(
    r"^m(\d+)xn(\d+)xk(\d+)"
    r"_wg(\d+)x(\d+)x(\d+)_w(\d+)x(\d+)x(\d+)"
    r"_twg(\d+)x(\d+)x(\d+)_pipestrat(\d+)"
    r"_wgcu(\d+)_lcm([01])_um(\d+)_epeel([01])_llsched(\d+)_hoistwait([01])_rotc([01])"
    r"(?:_consbar([01]))?"
    r"_lt_(flat|buf)$"
)


class WeakScaledMappedGemmInstance:
    """A validated (spec, mapping) pair with label serde (gemm_config.py:509-719)."""

    _KERNEL_NAMES = {
        OperandPath.LDS: "gemm_f16_weak_scaled",
        OperandPath.DIRECT_B: "gemm_f16_direct_b",
        OperandPath.DIRECT_AB: "gemm_f16_direct_ab",
    }

    def __init__(self, spec: GemmSpec, mapping: GemmMappingSpec):
        self.spec = spec
        self.mapping = mapping
        self._check_weak_scale()

    def _check_weak_scale(self) -> None:
        wg, twg = self.mapping.num_workgroups_per_kernel, self.mapping.num_tiles_per_workgroup
        size, mfma = self.spec.gemm_size, self.spec.mfma_shape
        for dim, name in ((DIM_M, "M"), (DIM_N, "N")):
            expected = wg[dim] * twg[dim] * mfma[dim]
            assert size[dim] == expected, (
                f"gemm_size[{name}]={size[dim]} != num_workgroups_per_kernel[{name}]({wg[dim]}) * "
                f"num_tiles_per_wg[{name}]({twg[dim]}) * mfma_shape[{name}]({mfma[dim]}) = {expected}"
            )

    @property
    def gemm_size(self) -> list[int]:
        return self.spec.gemm_size

    @property
    def load_type(self) -> str:
        return self.mapping.load_type.value

    @property
    def b_path(self) -> str:
        return self.mapping.operand_path.value

    @property
    def estimated_agprs(self) -> int:
        return self.mapping.estimated_agprs()

    @property
    def estimated_vgprs(self) -> int:
        return self.mapping.estimated_vgprs()

    @property
    def lds_bytes(self) -> int:
        return self.mapping.lds_bytes()

    @property
    def simd_occupancy(self) -> int:
        return self.mapping.simd_occupancy()

    @property
    def kernel_name(self) -> str:
        return self._KERNEL_NAMES[self.mapping.operand_path]

    @property
    def k_scaling_factor(self) -> int:
        tile_k = self.mapping.tile_elements(self.spec.mfma_shape)[DIM_K]
        return self.gemm_size[DIM_K] // (self.mapping.num_tiles_per_wave[DIM_K] * tile_k)

    # --- label serde: every pinnable knob is written explicitly, round-trip is exact ---
    @classmethod
    def _label_pattern(cls):
        return _LABEL_RE

    @classmethod
    def _parts_from_label(cls, label: str) -> tuple[GemmSpec, GemmMappingSpec]:
        m = _LABEL_RE.match(label)
        if not m:
            raise ValueError(f"Cannot parse label: {label}")
        g = m.groups()
        size = [int(v) for v in g[0:3]]
        wg = [int(v) for v in g[3:6]]
        waves = [int(v) for v in g[6:9]]
        twg = [int(v) for v in g[9:12]]
        pipestrat, wgcu, lcm, um, epeel, llsched, hoistwait, rotc, consbar, lt = g[12:]
        spec = GemmSpec.from_sizes(*size)
        mapping = GemmMappingSpec(
            num_workgroups_per_kernel=wg,
            num_waves_per_workgroup=waves,
            num_tiles_per_wave=[t // w for t, w in zip(twg, waves)],
            pipeline_strategy=int(pipestrat),
            load_type=LoadType.BUFFER if lt == "buf" else LoadType.FLAT,
            num_wg_per_cu=int(wgcu),
            lcm_unroll=lcm == "1",
            unroll_factor_multiplier=int(um),
            epilogue_peeling=epeel == "1",
            ll_sched=int(llsched),
            hoist_wait=hoistwait == "1",
            rotate_compute_stage=rotc == "1",
            use_conservative_barriers=consbar == "1",
        )
        return spec, mapping

    @classmethod
    def from_label(cls, label: str, strict: bool = True) -> "WeakScaledMappedGemmInstance":
        """Parse a label.  Like the reference, the result must serialise back to exactly
        ``label``; ``strict=False`` waives that for labels written before ``_consbar`` became
        mandatory (every entry of the reference's best_known.json is such a label)."""
        cfg = cls(*cls._parts_from_label(label))
        assert not strict or cfg.label == label, f"Round-trip failed: {cfg.label!r} != {label!r}"
        return cfg

    @property
    def label(self) -> str:
        m = self.mapping
        size, wg, waves, twg = self.gemm_size, m.num_workgroups_per_kernel, m.num_waves_per_workgroup, self.num_tiles_per_workgroup
        triple = lambda v: "x".join(str(x) for x in v)  # noqa: E731
        return (
            f"m{size[DIM_M]}xn{size[DIM_N]}xk{size[DIM_K]}"
            f"_wg{triple(wg)}_w{triple(waves)}_twg{triple(twg)}"
            f"_pipestrat{m.pipeline_strategy}_wgcu{m.num_wg_per_cu}"
            f"_lcm{int(m.lcm_unroll)}_um{m.unroll_factor_multiplier}_epeel{int(m.epilogue_peeling)}"
            f"_llsched{int(m.ll_sched)}_hoistwait{int(m.hoist_wait)}_rotc{int(m.rotate_compute_stage)}"
            f"_consbar{int(m.use_conservative_barriers)}"
            f"_lt_{'buf' if m.load_type == LoadType.BUFFER else 'flat'}"
        )

    def __getattr__(self, name: str):
        # Delegate to spec, then mapping.  `spec`/`mapping` themselves may be absent while
        # unpickling, so never recurse on them.
        if name in ("spec", "mapping"):
            raise AttributeError(name)
        for owner in ("spec", "mapping"):
            try:
                return getattr(object.__getattribute__(self, owner), name)
            except AttributeError:
                continue
        raise AttributeError(f"'{type(self).__name__}' has no attribute '{name}'") from None


# ---------------------------------------------------------------------------------------------
# B200 reading of an instance
# ---------------------------------------------------------------------------------------------
_ELT_BYTES = {"f16": 2, "bf16": 2, "e4m3": 1, "e5m2": 1, "i8": 1, "f32": 4, "i32": 4}
_LEGAL_TILE_N = (256, 128, 64, 32)
_B200_SUFFIX_RE = re.compile(
    r"_b200_(f16|bf16|e4m3|e5m2|i8)_o(f32|bf16|i32)_e(none|biasrelu|bias|relu)(_bm)?(?:_bn(\d+))?(?:_st(\d+))?(?:_sk(-?\d+))?(?:_cg(\d))?$"
)
_EPI_TOKEN = {"none": "none", "bias_relu": "biasrelu", "bias": "bias", "relu": "relu"}
_EPI_FROM_TOKEN = {v: k for k, v in _EPI_TOKEN.items()}


def strip_target_suffix(label: str) -> str:
    """Drop the ``_cdna4`` marker the reference appends to gfx950 labels before parsing
    (test_102_gemm_python_multitile_g2s_directb_cdna4.py:369-384)."""
    return label[: -len("_cdna4")] if label.endswith("_cdna4") else label


class B200GemmInstance(WeakScaledMappedGemmInstance):
    """An instance plus what the reference label cannot say: element types, epilogue and the
    B200 tile overrides.  Plays the role of the reference's ``MultitileGemmInstance``
    (test_102_gemm_python_multitile_lds_cdna3.py:360-388).

    The extras travel as a suffix after ``_lt_{flat|buf}`` -- the same device the reference
    uses for its ``_cdna4`` labels (test_102_..._g2s_directb_cdna4.py:369-384) -- so a plain
    reference label parses to the defaults (f16 in, f32 out, no epilogue).
    """

    KERNEL_NAME = "gemm_multitile"

    def __init__(self, spec: GemmSpec, mapping: GemmMappingSpec, *, dtype_ab: str = "f16", dtype_c: str = "f32",
                 epilogue: str = "none", bias_axis: str = "n", tile_n: int = 0, stages: Optional[int] = None, split_k: int = 0,
                 cta_group: int = 0):
        super().__init__(spec, mapping)
        if dtype_ab not in ("f16", "bf16", "e4m3", "e5m2", "i8") or dtype_c not in ("f32", "bf16", "i32") or (
                dtype_c == "i32" and dtype_ab != "i8"):
            raise ValueError(f"unsupported element types {dtype_ab!r} -> {dtype_c!r}")
        if epilogue not in _EPI_TOKEN:
            raise ValueError(f"unknown epilogue {epilogue!r}")
        if spec.elt_bytes_a != _ELT_BYTES[dtype_ab] or spec.elt_bytes_b != _ELT_BYTES[dtype_ab]:
            raise ValueError(f"spec element width {spec.elt_bytes_a} does not match dtype {dtype_ab}")
        if spec.elt_bytes_c != _ELT_BYTES[dtype_c]:
            raise ValueError(f"spec output width {spec.elt_bytes_c} does not match dtype {dtype_c}")
        self.dtype_ab, self.dtype_c = dtype_ab, dtype_c
        self.epilogue, self.bias_axis = epilogue, bias_axis
        self.tile_n_override = int(tile_n)
        self.stages_override = None if stages is None else int(stages)  # None: from the pipeline strategy; 0: as many as fit
        self.split_k, self.cta_group = int(split_k), int(cta_group)

    @property
    def kernel_name(self) -> str:
        return self.KERNEL_NAME

    # transfer-tile geometry of the reference instance (test_102_...:372-388)
    @property
    def transfer_tile_k_elems(self) -> int:
        return (self.mapping.wave_size // self.spec.mfma_shape[DIM_M]) * (self.mapping.global_load_bytes // self.spec.elt_bytes_a)

    @property
    def transfer_tile_row_bytes(self) -> int:
        return self.transfer_tile_k_elems * self.spec.elt_bytes_a

    @property
    def transfer_tile_bytes(self) -> int:
        return self.spec.mfma_shape[DIM_M] * self.transfer_tile_row_bytes

    # --- B200 mapping ---
    @property
    def requested_cta_tile(self) -> list[int]:
        """``[twg_m * 16, twg_n * 16, twg_k * 32]``: the workgroup tile the label asks for."""
        te = self.mapping.tile_elements(self.spec.mfma_shape)
        return [t * e for t, e in zip(self.mapping.num_tiles_per_workgroup, te)]

    @property
    def tile_n(self) -> int:
        """CTA tile width: the override, else the widest legal width <= the requested one."""
        if self.tile_n_override:
            return self.tile_n_override
        want = self.requested_cta_tile[DIM_N]
        for legal in _LEGAL_TILE_N:
            if legal <= want:
                return legal
        return _LEGAL_TILE_N[-1]

    @property
    def stages(self) -> int:
        """Shared-memory ring depth handed to the plan: the ``_st`` override when the label has
        one (``_st0`` = as many slots as fit in shared memory), else the pipeline strategy's
        depth ``max(stage) + 1``."""
        return self.mapping.pipeline_depth if self.stages_override is None else self.stages_override

    def plan_kwargs(self) -> dict:
        """Arguments for :class:`aster_b200.gemm.GemmPlan`."""
        m, n, k = self.gemm_size
        b_layout = "ref_preshuffled" if self.mapping.direct_b else "row_major"
        return dict(
            M=m, N=n, K=k, dtype_ab=self.dtype_ab, dtype_c=self.dtype_c, b_layout=b_layout, epilogue=self.epilogue,
            bias_axis=self.bias_axis, tile_n=self.tile_n, stages=self.stages, split_k=self.split_k,
            cta_group=self.cta_group, label=self.label,
        )

    @property
    def b200_suffix(self) -> str:
        s = f"_b200_{self.dtype_ab}_o{self.dtype_c}_e{_EPI_TOKEN[self.epilogue]}"
        if self.bias_axis == "m":
            s += "_bm"
        if self.tile_n_override:
            s += f"_bn{self.tile_n_override}"
        if self.stages_override is not None:
            s += f"_st{self.stages_override}"
        if self.split_k:
            s += f"_sk{self.split_k}"
        if self.cta_group:
            s += f"_cg{self.cta_group}"
        return s

    @property
    def is_plain(self) -> bool:
        return (self.dtype_ab, self.dtype_c, self.epilogue, self.bias_axis) == ("f16", "f32", "none", "n") and not (
            self.tile_n_override or self.stages_override is not None or self.split_k or self.cta_group
        )

    @property
    def label(self) -> str:
        base = WeakScaledMappedGemmInstance.label.fget(self)
        return base if self.is_plain else base + self.b200_suffix

    @classmethod
    def from_label(cls, label: str, operand_path: OperandPath = OperandPath.LDS, strict: bool = True) -> "B200GemmInstance":
        extras = {}
        label = strip_target_suffix(label)
        base = label
        sm = _B200_SUFFIX_RE.search(label)
        if sm:
            base = label[: sm.start()]
            dt_ab, dt_c, epi, bm, bn, st, sk, cg = sm.groups()
            extras = dict(dtype_ab=dt_ab, dtype_c=dt_c, epilogue=_EPI_FROM_TOKEN[epi], bias_axis="m" if bm else "n",
                          tile_n=int(bn or 0), stages=None if st is None else int(st), split_k=int(sk or 0), cta_group=int(cg or 0))
        spec, mapping = cls._parts_from_label(base)
        if extras:
            m, n, k = spec.gemm_size
            eb = _ELT_BYTES[extras["dtype_ab"]]
            spec = GemmSpec.from_sizes(m, n, k, elt_bytes_a=eb, elt_bytes_b=eb, elt_bytes_c=_ELT_BYTES[extras["dtype_c"]])
        mapping.operand_path = operand_path
        cfg = cls(spec, mapping, **extras)
        assert not strict or cfg.label == label, f"Round-trip failed: {cfg.label!r} != {label!r}"
        return cfg


def make_b200_instance(M: int, N: int, K: int, *, dtype_ab: str = "f16", dtype_c: str = "f32", epilogue: str = "none",
                       bias_axis: str = "n", tile_n: int = 256, stages: Optional[int] = 0, split_k: int = 0, cta_group: int = 0,
                       operand_path: OperandPath = OperandPath.LDS, pipeline_strategy: int = 3) -> B200GemmInstance:
    """Build an instance for sizes that are multiples of 16, picking a workgroup grid whose
    tile is ``128 x tile_n`` when the sizes allow it (otherwise one workgroup spans the
    dimension), with the reference's usual 1x4 wave grid.  ``stages=0`` (default) lets the plan
    use as many ring slots as fit; ``stages=None`` derives the depth from the pipeline strategy
    and, with the other defaults, yields a plain reference label."""
    if M % 16 or N % 16:
        raise ValueError("the weak-scale identity needs M and N to be multiples of 16")

    def split(extent: int, tile: int) -> tuple[int, int]:
        tiles16 = extent // 16
        per = tile // 16
        return (tiles16 // per, per) if tiles16 % per == 0 else (1, tiles16)

    wg_m, twg_m = split(M, 128)
    wg_n, twg_n = split(N, tile_n)
    waves_n = 4 if twg_n % 4 == 0 else 1
    eb = _ELT_BYTES[dtype_ab]
    spec = GemmSpec.from_sizes(M, N, K, elt_bytes_a=eb, elt_bytes_b=eb, elt_bytes_c=_ELT_BYTES[dtype_c])
    mapping = GemmMappingSpec(
        num_workgroups_per_kernel=[wg_m, wg_n, 1],
        num_waves_per_workgroup=[1, waves_n, 1],
        num_tiles_per_wave=[twg_m, twg_n // waves_n, 1],
        pipeline_strategy=pipeline_strategy,
        operand_path=operand_path,
    )
    return B200GemmInstance(spec, mapping, dtype_ab=dtype_ab, dtype_c=dtype_c, epilogue=epilogue, bias_axis=bias_axis,
                            stages=stages, split_k=split_k, cta_group=cta_group)
