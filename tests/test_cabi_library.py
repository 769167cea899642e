"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and
validates plan descriptions with status codes instead of undefined behaviour."""

import ctypes as C
import os
import re

import pytest

from aster_b200 import _native as nat
from aster_b200.gemm import GemmPlan
from aster_b200.multitile_gemm import compile_multitile_gemm, fits_on_sm_post_compile, load_artifact
from aster_b200.gemm_config import make_b200_instance

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "aster_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_groups():
    names = declared_functions()
    assert len(names) >= 40
    for must in ("b200_init", "b200_malloc", "b200_gemm_plan_create", "b200_gemm_run", "b200_gemm_time",
                 "b200_pack_b", "b200_vector_add_i32", "b200_copy_2d_padded_f32", "b200_add_relu_f32", "b200_status_read"):
        assert must in names


def test_library_exports_every_declared_symbol(native_lib):
    missing = [n for n in declared_functions() if not hasattr(native_lib, n)]
    assert not missing, f"declared in include/aster_b200.h but not exported: {missing}"


def test_binding_covers_every_declared_symbol():
    bound = set(nat.SIGNATURES) | set(nat._NON_STATUS)
    assert set(declared_functions()) == bound


def test_struct_sizes_match_header_layout(native_lib):
    # int64 x3 + int32 x16 + char[256]; int32 x12 + int64 x4 + int32 x4; char[128] + int32 x10 + int64
    assert C.sizeof(nat.GemmDesc) == 24 + 64 + 256
    assert C.sizeof(nat.GemmResources) == 48 + 32 + 16
    assert C.sizeof(nat.Props) == 128 + 40 + 8


def test_version_and_error_text(native_lib):
    assert b"sm_100a" in native_lib.b200_version()
    assert native_lib.b200_device_reset() == nat.ERR_UNSUPPORTED
    assert "shared" in nat.last_error()
    assert native_lib.b200_malloc(None, 16) == nat.ERR_INVALID
    assert native_lib.b200_copy_2d_padded_f32(None, None, 4, 6, 2, 0, None) == nat.ERR_INVALID
    assert "multiple of 4" in nat.last_error()
    assert native_lib.b200_copy_2d_padded_f32(None, None, 4, 8, 9, 0, None) == nat.ERR_INVALID


@pytest.mark.parametrize("kw,fragment", [
    (dict(M=0, N=64, K=64), "must be >= 1"),
    (dict(M=64, N=64, K=7), "multiple of 16 bytes"),
    (dict(M=64, N=64, K=24, dtype_ab="e4m3"), "multiple of 16 bytes"),
    (dict(M=64, N=64, K=64, tile_n=48), "tile_n=48"),
    (dict(M=64, N=64, K=64, tile_m=64), "tile_m=64"),
    (dict(M=512, N=64, K=64, tile_m=128, cta_group=2), "contradicts"),
    (dict(M=512, N=64, K=64, cta_group=2, tile_n=32), "tile_n >= 64"),
    (dict(M=512, N=64, K=64, cta_group=2, b_layout="packed"), "cta_group=1"),
    (dict(M=64, N=64, K=64, stages=17), "stages=17"),
    (dict(M=64, N=64, K=64, tile_n=256, stages=5), "shared memory limit"),
    (dict(M=512, N=512, K=64, tile_n=256, stages=8, cta_group=2), "shared memory limit"),
    (dict(M=64, N=64, K=64, cta_group=3), "cta_group=3"),
    (dict(M=64, N=40, K=64, b_layout="ref_preshuffled"), "preshuffled"),
    (dict(M=64, N=64, K=64, split_k=65), "split_k"),
    (dict(M=1 << 31, N=64, K=64), "below 2^31"),
])
def test_plan_validation_returns_invalid(native_lib, kw, fragment):
    with pytest.raises(nat.B200Error) as e:
        GemmPlan(**kw)
    assert e.value.status == nat.ERR_INVALID and fragment in e.value.message


def test_plan_enum_validation(native_lib):
    desc = nat.GemmDesc(M=64, N=64, K=64, dtype_ab=7)
    handle = C.c_void_p()
    assert native_lib.b200_gemm_plan_create(C.byref(desc), C.byref(handle)) == nat.ERR_INVALID and not handle.value
    assert native_lib.b200_gemm_plan_create(None, C.byref(handle)) == nat.ERR_INVALID
    with pytest.raises(ValueError):
        GemmPlan(64, 64, 64, dtype_ab="int4")


def test_plan_resources_without_a_gpu(native_lib):
    p = GemmPlan(4096, 4096, 4096, "bf16", "bf16")
    r = p.resources()
    assert (r.tile_m, r.tile_n, r.tile_k, r.block_threads, r.cta_group) == (256, 256, 64, 192, 2)
    assert r.num_tiles == 16 * 16 and r.grid_ctas == 148 and r.tmem_columns == 512 and r.stages == 7
    single = GemmPlan(4096, 4096, 4096, "bf16", "bf16", cta_group=1).resources()
    assert (single.tile_m, single.cta_group, single.num_tiles, single.stages) == (128, 1, 32 * 16, 4)
    assert r.smem_bytes <= 232448 and r.ctas_per_sm == 1 and r.workspace_bytes == 0 and r.packed_b_bytes == 0
    p.destroy()
    p.destroy()  # idempotent
    small = GemmPlan(512, 512, 2048).resources()
    assert small.tile_n == 128 and small.num_tiles == 8 and small.cta_group == 2
    assert (small.tail_tiles, small.tail_parts, small.grid_ctas) == (8, 2, 32) and small.optional_workspace_bytes > 0
    short = GemmPlan(512, 512, 512).resources()  # too few K blocks to pay for the exchange; small single-CTA tiles for latency
    assert (short.tail_parts, short.optional_workspace_bytes) == (0, 0)
    assert (short.cta_group, short.tile_n, short.grid_ctas) == (1, 32, 64)
    # pairs pay per tile: at most 8 K blocks, or one round of 128 x 256 tiles on most SMs -> single CTAs
    for shape, want in [((8192, 8192, 512), (1, 256, 148)), ((2048, 2048, 2048), (1, 256, 128)), ((4096, 4096, 1024), (2, 256, 148)),
                        ((512, 8192, 8192), (2, 256, 128))]:
        got = GemmPlan(*shape, "bf16", "bf16").resources()
        assert (got.cta_group, got.tile_n, got.grid_ctas) == want, shape
    # 34 tiles x 2 parts: fp32 partial tiles of 256 x 256 plus one ready flag per epilogue warp, padded to 256 bytes
    assert (r.tail_tiles, r.tail_parts) == (34, 2)
    assert r.optional_workspace_bytes == 34 * 2 * 256 * 256 * 4 + -(-(34 * 2 * 2 * 4 * 4) // 256) * 256
    assert GemmPlan(8192, 8192, 8192, "bf16", "bf16").resources().tail_parts == 0
    fp8 = GemmPlan(256, 256, 1024, "e4m3", "bf16").resources()
    assert fp8.tile_k == 128
    skinny = GemmPlan(16, 8192, 8192, "bf16", "bf16", split_k=-1, tile_n=64).resources()
    assert skinny.split_k >= 1 and skinny.workspace_bytes == skinny.split_k * 16 * 8192 * 4 * (skinny.split_k > 1)
    packed = GemmPlan(256, 300 * 16, 512, b_layout="packed", tile_n=256).resources()
    assert packed.packed_b_bytes == 19 * 256 * 8 * 128 and packed.cta_group == 1


def test_run_argument_checks_do_not_need_a_gpu(native_lib):
    p = GemmPlan(128, 128, 128)
    with pytest.raises(nat.B200Error) as e:
        p.run(None, None, None)
    assert e.value.status == nat.ERR_INVALID
    with pytest.raises(nat.B200Error, match="16-byte aligned"):
        p.run(0x1008, 0x2000, 0x3000)
    p2 = GemmPlan(128, 128, 128, epilogue="bias_relu")
    with pytest.raises(nat.B200Error, match="needs a bias"):
        p2.run(0x1000, 0x2000, 0x3000)
    p3 = GemmPlan(16, 1024, 4096, split_k=4)
    with pytest.raises(nat.B200Error) as e3:
        p3.run(0x1000, 0x2000, 0x3000)
    assert e3.value.status == nat.ERR_WORKSPACE
    need = p3.resources().workspace_bytes
    with pytest.raises(nat.B200Error, match="workspace must be 16-byte aligned") as e4:  # refused on the host: nothing is launched
        p3.run(0x1000, 0x2000, 0x3000, workspace=0x100004, workspace_bytes=need)
    assert e4.value.status == nat.ERR_INVALID
    assert p.status() == [0, 0, 0, 0]  # never launched


def test_work_skipping_modes_are_not_in_the_default_build(native_lib):
    """reserved[0] accepts the wait-limit fault injection (8) and "no dependent launch" (16); the
    modes that make the kernel skip copies, multiplies or stores belong to the bring-up build."""
    GemmPlan(128, 128, 128, debug_mode=8 | 16).destroy()
    if nat.is_bringup_build():
        pytest.skip("bring-up library loaded")
    assert not hasattr(native_lib, "b200_gemm_debug_timeline")
    for mode in (1, 2, 4, 32, 64):
        with pytest.raises(nat.B200Error, match="B200_BRINGUP") as e:
            GemmPlan(128, 128, 128, debug_mode=mode)
        assert e.value.status == nat.ERR_INVALID


def test_noalloc_status_reads_zero_before_any_call(native_lib):
    words = (C.c_uint32 * 4)(7, 7, 7, 7)
    if nat.device_count() < 1:
        assert native_lib.b200_gemm_splitk_noalloc_status(words) != nat.OK  # no device to ask
        assert native_lib.b200_gemm_splitk_noalloc_status(None) == nat.ERR_INVALID
    else:
        assert native_lib.b200_gemm_splitk_noalloc_status(None) == nat.ERR_INVALID


def test_compile_fn_writes_an_artifact(tmp_path, native_lib):
    cfg = make_b200_instance(4096, 4096, 4096, dtype_ab="bf16", dtype_c="bf16")
    path, text = compile_multitile_gemm(cfg, str(tmp_path / "a.b200plan.json"), num_vgprs=256, print_asm=False)
    art = load_artifact(path)
    assert art["label"] == cfg.label and art["plan"]["tile_n"] == 256 and art["resources"]["tmem_columns"] == 512
    assert fits_on_sm_post_compile(cfg, art["resources"]) is None
    assert fits_on_sm_post_compile(cfg, dict(art["resources"], smem_bytes=300000)) is not None
    (tmp_path / "bad.json").write_text("{}")
    with pytest.raises(RuntimeError):
        load_artifact(str(tmp_path / "bad.json"))


def test_older_template_family_entry_points(tmp_path, native_lib):
    """compile_gemm / execute_gemm_hsaco of test_perf_001 accept the plain config type."""
    from aster_b200.gemm_config import GemmMappingSpec, GemmSpec, WeakScaledMappedGemmInstance
    from aster_b200.multitile_gemm import compile_gemm, execute_gemm_hsaco  # noqa: F401

    plain = WeakScaledMappedGemmInstance(GemmSpec.from_sizes(256, 256, 128), GemmMappingSpec([2, 2, 1], [2, 2, 1], [4, 4, 1]))
    path, text = compile_gemm(plain, str(tmp_path / "w.b200plan.json"), num_vgprs=256, num_agprs=256)
    art = load_artifact(path)
    assert art["label"].startswith(plain.label) and art["plan"]["M"] == 256 and art["kernel_name"] == "gemm_multitile"


def test_nccl_entry_points_check_arguments_without_a_gpu(native_lib):
    """NCCL is opened at run time: with it present the version reads back, without it the call
    says so; argument checks come before any NCCL or CUDA call."""
    import ctypes as C

    v = C.c_int(0)
    rc = native_lib.b200_nccl_version(C.byref(v))
    if rc == nat.OK:
        assert v.value >= 20000
    else:
        assert rc == nat.ERR_UNSUPPORTED and b"NCCL runtime not available" in native_lib.b200_last_error()
    comm = C.c_void_p(123)
    assert native_lib.b200_nccl_init_all(0, None, C.byref(comm)) == nat.ERR_INVALID and comm.value is None
    assert b"ndev 0 out of range" in native_lib.b200_last_error()
    assert native_lib.b200_nccl_destroy(None) == nat.OK
    assert native_lib.b200_allgather_rows(None, 0, None, None, 16, None) == nat.ERR_INVALID
    assert b"comm is NULL" in native_lib.b200_last_error()
