"""CPU tests of the drop-in boundary: fixture -> realization -> provider route -> plan ->
target export, driven through the tcrv-opt / tcrv-translate look-alikes.  Structure follows
the reference's lit tests: positive plan/header checks, fail-closed negatives (one edited
attribute each) and tamper tests that edit the materialised plan before export
(test/Target/RVV/pre-realized-selected-body-artifact-add.mlir:1-10 in the reference)."""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "tianchen-rv_b200")
FIX = os.path.join(PKG, "test", "fixtures")
OPT = os.path.join(PKG, "build", "bin", "tcrv-opt")
TRANSLATE = os.path.join(PKG, "build", "bin", "tcrv-translate")
PLAN_PASSES = ["--tcrv-check-capability-requires", "--tcrv-materialize-selected-lowering-boundaries",
               "--tcrv-materialize-emission-plans"]


@pytest.fixture(scope="module", autouse=True)
def tools():
    subprocess.run(["make", "-s", "-C", PKG], check=True)


def run(cmd, text):
    return subprocess.run(cmd, input=text, capture_output=True, text=True)


def fixture(name):
    return open(os.path.join(FIX, name)).read()


def plan(text, passes=PLAN_PASSES):
    r = run([OPT, "-", *passes], text)
    assert r.returncode == 0, r.stderr
    return r.stdout


def header(plan_text):
    return run([TRANSLATE, "-", "--tcrv-export-target-header-artifact"], plan_text)


PROTOTYPES = {
    "cuda-add-f32.mlir": "void tcrv_emitc_explicit_selected_body_add_f32_kernel_explicit_selected_body_cuda_f32_add("
                         "const float *lhs, const float *rhs, float *out, size_t n);",
    "cuda-add-i32.mlir": "void tcrv_emitc_explicit_selected_body_add_kernel_explicit_selected_body_rvv_i32_add("
                         "const int32_t *lhs, const int32_t *rhs, int32_t *out, size_t n);",
    "cuda-dequantize-i32-to-f32.mlir":
        "void tcrv_emitc_explicit_selected_body_dequantize_i32_to_f32_kernel_explicit_selected_body_rvv_dequantize_i32_to_f32("
        "const int32_t *lhs, float scale, float *out, size_t n);",
    "cuda-quantize-row-q8-0.mlir": "void tcrv_emitc_quantize_row_q8_0_kernel_quantize_row_q8_0("
                                   "size_t n, const float *x, uint8_t *vy);",
    "cuda-ggml-vec-scale-f32.mlir": "void tcrv_emitc_ggml_vec_scale_f32_kernel_ggml_vec_scale_f32("
                                    "size_t n, float *y, float v);",
    "cuda-ggml-rms-norm-f32.mlir": "void tcrv_emitc_ggml_rms_norm_f32_kernel_ggml_rms_norm_f32("
                                   "size_t ne00, const float *x, float *y, float eps);",
    "cuda-ggml-vec-silu-f32.mlir": "void tcrv_emitc_ggml_vec_silu_f32_kernel_ggml_vec_silu_f32("
                                   "size_t n, const float *x, float *y);",
    "cuda-ggml-vec-soft-max-f32.mlir": "double tcrv_emitc_ggml_vec_soft_max_f32_kernel_ggml_vec_soft_max_f32("
                                       "size_t n, float *y, const float *x, float max);",
    "cuda-ggml-rope-norm-f32.mlir": "void tcrv_emitc_ggml_rope_norm_f32_kernel_ggml_rope_norm_f32("
                                    "size_t n_dims, const float *x, float *y, float theta_base, float theta_scale);",
    "cuda-pack-q4-0-to-q4-0x16.mlir": "void tcrv_emitc_ggml_pack_q4_0_to_q4_0x16_kernel_ggml_pack_q4_0_to_q4_0x16("
                                      "size_t nblocks, const uint8_t *src, uint8_t *dst);",
    "cuda-q4-0-q8-0-integer-core.mlir":
        "void tcrv_emitc_rvv_q4_0_q8_0_integer_core_kernel_rvv_q4_0_q8_0_integer_core("
        "const int8_t *w, const int8_t *qlo, const int8_t *qhi, const int32_t *acc, int32_t *out, size_t n);",
    "cuda-q4-0-q8-0-gemm-tile.mlir": "void tcrv_emitc_ggml_q4_0_q8_0_gemm_tile_kernel_ggml_q4_0_q8_0_gemm_tile("
                                     "size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by);",
    "cuda-repack-gemv-q4-0-q8-0.mlir":
        "void tcrv_emitc_ggml_repack_gemv_q4_0_q8_0_kernel_ggml_repack_gemv_q4_0_q8_0("
        "size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc);",
    "cuda-repack-gemv-q8-0-q8-0.mlir":
        "void tcrv_emitc_ggml_repack_gemv_q8_0_q8_0_kernel_ggml_repack_gemv_q8_0_q8_0("
        "size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc);",
    "cuda-repack-gemm-q4-0-q8-0.mlir":
        "void tcrv_emitc_ggml_repack_gemm_q4_0_q8_0_kernel_ggml_repack_gemm_q4_0_q8_0("
        "size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nr, size_t nc, size_t bs);",
    "cuda-q4-1-q8-1-block-dot.mlir": "void tcrv_emitc_ggml_vec_dot_q4_1_q8_1_kernel_ggml_vec_dot_q4_1_q8_1("
        "size_t n, float *s, const uint8_t *vx, const uint8_t *vy);",
    "cuda-q5-0-q8-0-block-dot.mlir": "void tcrv_emitc_ggml_vec_dot_q5_0_q8_0_kernel_ggml_vec_dot_q5_0_q8_0("
        "size_t n, float *s, const uint8_t *vx, const uint8_t *vy);",
    "cuda-q5-1-q8-1-block-dot.mlir": "void tcrv_emitc_ggml_vec_dot_q5_1_q8_1_kernel_ggml_vec_dot_q5_1_q8_1("
        "size_t n, float *s, const uint8_t *vx, const uint8_t *vy);",
    "cuda-q4-0-q8-0-block-dot.mlir": "void tcrv_emitc_ggml_vec_dot_q4_0_q8_0_kernel_ggml_vec_dot_q4_0_q8_0("
                                     "size_t n, float *s, size_t bs, const uint8_t *vx, size_t bx, const uint8_t *vy, "
                                     "size_t by, int32_t nrc);",
    "cuda-q8-0-q8-0-block-dot.mlir": "void tcrv_emitc_ggml_vec_dot_q8_0_q8_0_kernel_ggml_vec_dot_q8_0_q8_0("
                                     "size_t n, float *s, const uint8_t *vx, const uint8_t *vy);",
    "cuda-q4-0-q8-0-gemm.mlir": "void tcrv_emitc_ggml_q4_0_q8_0_gemm_kernel_ggml_q4_0_q8_0_gemm("
                                "size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, "
                                "size_t nc, size_t bx, size_t bs);",
}


@pytest.mark.parametrize("name", sorted(PROTOTYPES))
def test_plan_and_header_for_every_fixture(name):
    p = plan(fixture(name))
    assert "tcrv.exec.diagnostic" in p and 'reason = "emission_plan"' in p and 'status = "supported"' in p
    assert 'artifact_kind = "cuda-sm100a-launch-descriptor"' in p
    assert 'emission_kind = "prebuilt-sm100a-kernel-c-abi-launch"' in p
    assert 'lowering_boundary = "tcrv_rvv.with_vl"' in p and 'origin = "cuda-plugin"' in p
    h = header(p)
    assert h.returncode == 0, h.stderr
    assert PROTOTYPES[name] in h.stdout
    assert "// tianchenrv.cuda.route_mapping: cuda-sm100a-typed-body-launch-route-family" in h.stdout
    assert "// tianchenrv.cuda.target_arch: sm_100a" in h.stdout
    # the entry name is derived, never configured: tcrv_emitc_<kernel>_<variant>
    assert "tcrv_emitc_" in h.stdout


def test_every_exported_entry_symbol_exists_in_the_library(pkg):
    import ctypes

    pkg.build_library()
    lib = ctypes.CDLL(pkg.LIB_PATH)
    for name in PROTOTYPES:
        p = plan(fixture(name))
        d = run([TRANSLATE, "-", "--tcrv-export-target-artifact"], p)
        assert d.returncode == 0, d.stderr
        desc = json.loads(d.stdout)
        assert desc["library"] == "libtcrv_cuda.so"
        assert hasattr(lib, desc["entry_symbol"]), desc["entry_symbol"]
        for launcher in desc["launcher_symbol"].split("|"):
            assert hasattr(lib, launcher), launcher
        assert hasattr(lib, desc["metadata"]["tcrv_cuda.host_pointer_symbol"])


def test_add_plan_records_role_facts_and_abi_order():
    p = plan(fixture("cuda-add-f32.mlir"))
    assert 'role = "dispatch case"' in p
    assert 'runtime_abi_name = "cuda-generic-binary-add-f32-callable-c-abi.v1"' in p
    assert '"cuda_selected_body_operation=add"' in p and '"cuda_selected_body_typed_compute_op=tcrv_rvv.binary"' in p
    assert '"tcrv_cuda.element_type=f32"' in p
    assert ('abi_parameters = ["lhs|const float *|lhs-input-buffer|target-export-abi-owned", '
            '"rhs|const float *|rhs-input-buffer|target-export-abi-owned", '
            '"out|float *|output-buffer|target-export-abi-owned", '
            '"n|size_t|runtime-element-count|target-export-abi-owned"]') in p
    m = run([TRANSLATE, "-", "--tcrv-export-emission-manifest"], p)
    assert m.returncode == 0 and "launcher=tcrv_cuda_add_f32" in m.stdout and 'role="dispatch case"' in m.stdout


@pytest.mark.parametrize("extra", [
    'integer_core_lmul = "m1"',
    'integer_core_lmul = "m1", multi_block_factor = 2 : i64, strip_elision = "robust"',
    'integer_core_lmul = "m1", multi_block_factor = 4 : i64, strip_elision = "elided"',
])
def test_block_dot_schedule_attributes_of_the_rvv_variants_are_accepted(extra):
    # the reference's -m1 / -mb2-robust / -mb4-elided fixtures differ from the base block dot only in
    # attributes that choose HOW the RVV kernel is scheduled; they do not select another kernel here
    src = fixture("cuda-q4-0-q8-0-block-dot.mlir")
    anchor = "activation_high_byte_offset = 16 : i64"
    assert anchor in src
    p = plan(src.replace(anchor, anchor + ", " + extra))
    assert 'status = "supported"' in p and 'runtime_abi_name = "cuda-ggml-q4_0-q8_0-block-dot-callable-c-abi.v1"' in p


def test_gemm_tile_column_count_is_a_checked_compile_time_argument():
    src = fixture("cuda-q4-0-q8-0-gemm-tile.mlir")
    p = plan(src)
    assert '"tcrv_cuda.constant_arguments=activation_cols=4"' in p
    # another column count: the generated entry passes it to the host-pointer call as a literal
    p7 = plan(src.replace("activation_cols = 4", "activation_cols = 7"))
    stub = run([TRANSLATE, "-", "--tcrv-cuda-launch-to-cpp"], p7)
    assert stub.returncode == 0, stub.stderr
    assert "tcrv_cuda_host_gemm_tile_q4_0_q8_0(n, s, vx, vy, by, /*activation_cols=*/7);" in stub.stdout
    for bad in ("activation_cols = 0", "activation_cols = 17"):
        r = run([OPT, "-", *PLAN_PASSES], src.replace("activation_cols = 4", bad))
        assert r.returncode != 0 and "'activation_cols' must lie in 1..16" in r.stderr, r.stderr
    r = run([OPT, "-", *PLAN_PASSES], src.replace(", activation_cols = 4 : i64", ""))
    assert r.returncode != 0 and "missing integer attribute 'activation_cols'" in r.stderr, r.stderr


def test_gemm_plan_pins_block_format_facts():
    p = plan(fixture("cuda-q4-0-q8-0-gemm.mlir"))
    assert ("tcrv_cuda.typed_facts=kind=ggml_q4_0_q8_0_gemm;scale_model=dual-fp16-per-block-d_x.d_y;qk=32;"
            "weight_block_stride=18;activation_block_stride=34;quant_byte_offset=2;activation_high_byte_offset=16") in p
    assert "tcrv_cuda.launcher_symbol=tcrv_cuda_gemv_q4_0_q8_0|tcrv_cuda_gemm_q4_0_q8_0" in p
    assert 'role = "direct call"' in p


def test_pre_realized_body_is_realized_then_planned():
    src = fixture("cuda-add-f32-pre-realized.mlir")
    realized = plan(src, ["--tcrv-materialize-selected-lowering-boundaries"])
    assert "typed_binary_pre_realized_body" not in realized
    for needle in ('tcrv_rvv.setvl %n {lmul = "m1"', "tcrv_rvv.with_vl %vl attributes", 'origin = "cuda-plugin"',
                   'selected_path_role = "dispatch case"', "selected_variant = @pre_realized_body_cuda_f32_add",
                   'kind = "add"', "tcrv_rvv.store %out, %sum, %vl"):
        assert needle in realized, needle
    assert realized.count("tcrv_rvv.load") == 2
    h = header(plan(src))
    assert h.returncode == 0, h.stderr
    assert "void tcrv_emitc_pre_realized_body_add_f32_kernel_pre_realized_body_cuda_f32_add(const float *lhs" in h.stdout
    # realization is idempotent and the realized text parses again
    again = plan(realized, ["--tcrv-materialize-selected-lowering-boundaries"])
    assert again == realized
    # without realization there is no boundary to plan from
    r = run([OPT, "-", "--tcrv-materialize-emission-plans"], src)
    assert r.returncode != 0 and "expected exactly one tcrv_rvv.with_vl boundary" in r.stderr


def test_printer_round_trips():
    for name in PROTOTYPES:
        once = plan(fixture(name), [])
        assert plan(once, []) == once


NEGATIVES = [
    ("cuda-add-f32.mlir", 'status = "available"}\n    tcrv.exec.capability @scalar', 'status = "missing"}\n    tcrv.exec.capability @scalar',
     "is not available"),
    ("cuda-add-f32.mlir", "requires = [@cuda], tcrv_rvv.policy", "requires = [@gpu], tcrv_rvv.policy", "is not declared in the kernel"),
    ("cuda-add-f32.mlir", "requires = [@cuda], tcrv_rvv.policy", "requires = [], tcrv_rvv.policy", "non-empty 'requires'"),
    ("cuda-add-f32.mlir", 'id = "cuda.sm_100a"', 'id = "cuda.sm_90a"', "must require a capability"),
    ("cuda-add-f32.mlir", 'ownership = "target-export-abi-owned", purpose = "out"', 'ownership = "kernel-owned", purpose = "out"',
     "ownership must be"),
    ("cuda-add-f32.mlir", 'c_name = "rhs"', 'c_name = "lhs"', "used twice"),
    ("cuda-add-f32.mlir", 'c_name = "out"', 'c_name = "out buffer"', "not a safe C identifier"),
    ("cuda-add-f32.mlir", 'c_type = "float *"', 'c_type = "const float *"', "not allowed for role"),
    ("cuda-add-f32.mlir", 'c_type = "float *"', 'c_type = "double *"', "must be {output-buffer, float *}"),
    ("cuda-add-f32.mlir", 'source_kernel = "explicit_selected_body_add_f32_kernel"', 'source_kernel = "other"', "'source_kernel'"),
    ("cuda-add-f32.mlir", 'status = "selected-lowering-boundary"', 'status = "proposed"', "'status'"),
    ("cuda-add-f32.mlir", 'selected_path_role = "dispatch case"', 'selected_path_role = "direct call"', "'selected_path_role'"),
    ("cuda-add-f32.mlir", "selected_variant = @explicit_selected_body_cuda_f32_add", "selected_variant = @someone_else", "'selected_variant'"),
    ("cuda-add-f32.mlir", "required_capabilities = [@cuda]", "required_capabilities = [@scalar_fallback]", "'required_capabilities'"),
    ("cuda-add-f32.mlir", 'cuda_construction_protocol = "extension-family-construction-protocol.v1"',
     'cuda_construction_protocol = "extension-family-construction-protocol.v0"', "cuda_construction_protocol"),
    ("cuda-add-f32.mlir", '{kind = "add"}', '{kind = "sub"}', "'kind' must be \"add\""),
    ("cuda-add-f32.mlir", "tcrv_rvv.store %out, %sum", "tcrv_rvv.store %lhs, %sum", "must write the output buffer"),
    ("cuda-q4-0-q8-0-gemm.mlir", "weight_block_stride = 18", "weight_block_stride = 20", "'weight_block_stride' must be 18"),
    ("cuda-q4-0-q8-0-gemm.mlir", "activation_high_byte_offset = 16", "activation_high_byte_offset = 0", "'activation_high_byte_offset' must be 16"),
    ("cuda-q4-0-q8-0-gemm.mlir", "qk = 32", "qk = 64", "'qk' must be 32"),
    ("cuda-q4-0-q8-0-gemm.mlir", 'scale_model = "dual-fp16-per-block-d_x.d_y"', 'scale_model = "single-fp32"', "'scale_model'"),
    ("cuda-q4-0-q8-0-gemm.mlir", "tcrv_rvv.q4_0_q8_0_gemm %vx, %vy", "tcrv_rvv.q4_0_q8_0_gemm %vy, %vx", "operand #0 must be the lhs-input-buffer"),
    ("cuda-q8-0-q8-0-block-dot.mlir", "weight_block_stride = 34", "weight_block_stride = 18", "'weight_block_stride' must be 34"),
    ("cuda-quantize-row-q8-0.mlir", "block_stride = 34", "block_stride = 36", "'block_stride' must be 34"),
    # the interleaved layouts are pinned fact by fact, as the reference's verifiers pin them
    ("cuda-repack-gemv-q4-0-q8-0.mlir", "weight_block_stride = 288", "weight_block_stride = 144", "'weight_block_stride' must be 288"),
    ("cuda-repack-gemv-q4-0-q8-0.mlir", "weight_quant_byte_offset = 32", "weight_quant_byte_offset = 2", "'weight_quant_byte_offset' must be 32"),
    ("cuda-repack-gemv-q8-0-q8-0.mlir", "weight_block_stride = 544", "weight_block_stride = 288", "'weight_block_stride' must be 544"),
    ("cuda-repack-gemv-q8-0-q8-0.mlir", "weight_interleave = 16", "weight_interleave = 8", "'weight_interleave' must be 16"),
    ("cuda-repack-gemm-q4-0-q8-0.mlir", "activation_block_stride = 136", "activation_block_stride = 34", "'activation_block_stride' must be 136"),
    ("cuda-repack-gemm-q4-0-q8-0.mlir", "activation_interleave = 4", "activation_interleave = 8", "'activation_interleave' must be 4"),
    ("cuda-repack-gemm-q4-0-q8-0.mlir", 'role = "output-stride"', 'role = "lhs-input-stride"', "must be {output-stride, size_t}"),
    ("cuda-q4-0-q8-0-integer-core.mlir", 'product_relation = "offset-binary-i4mf4-x-i8mf4x2-to-i16mf2"',
     'product_relation = "twos-complement"', "'product_relation' must be"),
    ("cuda-q4-0-q8-0-integer-core.mlir", 'c_type = "const int32_t *"', 'c_type = "const float *"',
     "must be {accumulator-input-buffer, const int32_t *}"),
    ("cuda-q4-0-q8-0-block-dot.mlir", "tcrv_rvv.q4_0_q8_0_block_dot", "tcrv_rvv.iq4_nl_q8_0_block_dot", "no kernel for op"),
]


@pytest.mark.parametrize("name,old,new,message", NEGATIVES)
def test_fail_closed_negatives(name, old, new, message):
    src = fixture(name)
    assert old in src
    r = run([OPT, "-", *PLAN_PASSES], src.replace(old, new))
    assert r.returncode != 0
    assert message in r.stderr, r.stderr
    assert r.stderr.count("\n") == 1  # one-line diagnostic


def test_parse_errors_are_reported_with_a_line():
    r = run([OPT, "-"], "module {\n  tcrv.exec.kernel @k {\n")
    assert r.returncode != 0 and "line" in r.stderr
    r = run([OPT, "-"], "func.func @f() {\n}\n")
    assert r.returncode != 0 and "expected a top-level 'module'" in r.stderr


TAMPERS = [
    ("cuda-generic-binary-add-f32-callable-c-abi.v1", "cuda-generic-binary-add-f64-callable-c-abi.v1", "runtime_abi_name"),
    ('"lhs|const float *|lhs-input-buffer|target-export-abi-owned", "rhs|', '"rhs|const float *|lhs-input-buffer|target-export-abi-owned", "lhs|',
     "abi parameter #0"),
    ("tcrv_cuda.element_type=f32", "tcrv_cuda.element_type=f16", "metadata 'tcrv_cuda.element_type'"),
    ("tcrv_cuda.launcher_symbol=tcrv_cuda_add_f32", "tcrv_cuda.launcher_symbol=tcrv_cuda_add_i32", "metadata 'tcrv_cuda.launcher_symbol'"),
    ('launcher_symbol = "tcrv_cuda_add_f32"', 'launcher_symbol = "my_own_kernel"', "launcher_symbol"),
    ("stddef.h,stdint.h", "stddef.h", "required_header_declarations"),
    ('role = "dispatch case", route_id', 'role = "direct call", route_id', "role"),
    ('entry_symbol = "tcrv_emitc_explicit_selected_body_add_f32_kernel_explicit_selected_body_cuda_f32_add"',
     'entry_symbol = "tcrv_emitc_renamed"', "entry_symbol"),
]


@pytest.mark.parametrize("old,new,message", TAMPERS)
def test_tampered_plans_are_refused_at_export(old, new, message):
    p = plan(fixture("cuda-add-f32.mlir"))
    assert old in p
    h = header(p.replace(old, new, 1))
    assert h.returncode != 0
    assert "stale emission plan" in h.stderr and message in h.stderr, h.stderr


def test_export_needs_a_plan_and_a_provider():
    src = fixture("cuda-add-f32.mlir")
    h = header(plan(src, []))
    assert h.returncode != 0 and "carries no emission plan" in h.stderr
    r = run([OPT, "-", "--tcrv-disable-builtin-plugins", *PLAN_PASSES], src)
    assert r.returncode != 0 and 'no provider named "cuda-plugin"' in r.stderr
    t = run([TRANSLATE, "-", "--tcrv-disable-builtin-plugins", "--tcrv-export-target-header-artifact"], plan(src))
    assert t.returncode != 0 and 'no provider named "cuda-plugin"' in t.stderr


def test_launch_stub_defines_the_reference_named_entry():
    p = plan(fixture("cuda-add-f32-pre-realized.mlir"))
    s = run([TRANSLATE, "-", "--tcrv-cuda-launch-to-cpp"], p)
    assert s.returncode == 0, s.stderr
    assert 'extern "C" void tcrv_emitc_pre_realized_body_add_f32_kernel_pre_realized_body_cuda_f32_add(' in s.stdout
    assert "tcrv_cuda_host_add_f32(lhs, rhs, out, n);" in s.stdout
    # the stub is valid C++ against the public headers
    c = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), "-x", "c++", "-"],
                       input=s.stdout, capture_output=True, text=True)
    assert c.returncode == 0, c.stderr


def test_repacked_gemv_plan_says_which_layout_is_native():
    # the interleaved layout is served as a compatibility path: the plan a scheduler reads says so
    # and names both summation orders
    p = plan(fixture("cuda-repack-gemv-q4-0-q8-0.mlir"))
    assert "tcrv_cuda.layout_note=compatibility path" in p and "plain block rows are the native layout" in p
    assert "strict ascending blocks (the reference's lane-wise chain)" in p
    assert "tcrv_cuda.layout_note" not in plan(fixture("cuda-q4-0-q8-0-gemm.mlir"))


def test_target_artifact_bundle_export_writes_files_and_index(tmp_path):
    # tcrv-export-target-artifact-bundle (reference driver, tools/tcrv-translate/tcrv-translate.cpp:40-48,
    # 469-474): one file per artifact plus the index, two lines on stdout
    p = plan(fixture("cuda-q4-0-q8-0-gemm.mlir"))
    out = tmp_path / "bundle"
    out.mkdir()
    r = run([TRANSLATE, "-", "--tcrv-export-target-artifact-bundle", f"--tcrv-target-artifact-bundle-output-dir={out}"], p)
    assert r.returncode == 0, r.stderr
    assert r.stdout == ('tianchenrv.target_artifact_bundle_export: complete\n'
                        'index_file: "tianchenrv-target-artifact-bundle.index"\n')
    names = sorted(os.listdir(out))
    obj = "artifact-0-cuda-sm100a-launch-descriptor-cuda-sm100a-typed-body-launch-route-family.json"
    hdr = "artifact-1-c-header-cuda-sm100a-typed-body-launch-route-family.h"
    assert names == [obj, hdr, "tianchenrv-target-artifact-bundle.index"]
    # the files are what the single-artifact exports print
    assert (out / hdr).read_text() == header(p).stdout
    assert (out / obj).read_text() == run([TRANSLATE, "-", "--tcrv-export-target-artifact"], p).stdout
    desc = json.loads((out / obj).read_text())
    assert "tcrv_cuda_gemm_q4_0_q8_0" in desc["launcher_symbol"].split("|")
    index = (out / "tianchenrv-target-artifact-bundle.index").read_text()
    for line in ["tianchenrv.target_artifact_bundle.version: 1", 'bundle_status: "complete"', "artifact_count: 2",
                 "artifact[0]:", f'  file_name: "{obj}"', '  component_role: "object"', "artifact[1]:",
                 f'  file_name: "{hdr}"', '  component_role: "header"',
                 "  selected_variant: @ggml_q4_0_q8_0_gemm", '  route: "cuda-sm100a-typed-body-launch-route-family"',
                 '  owner: "cuda-plugin"', "  runtime_abi_parameter_count: 9", '    c_name: "vx"',
                 '    ownership: "target-export-abi-owned"']:
        assert line in index.splitlines(), line


def test_target_artifact_bundle_export_fails_closed(tmp_path):
    p = plan(fixture("cuda-add-f32.mlir"))
    flag = "--tcrv-export-target-artifact-bundle"
    r = run([TRANSLATE, "-", flag], p)
    assert r.returncode != 0 and "--tcrv-target-artifact-bundle-output-dir is required" in r.stderr
    r = run([TRANSLATE, "-", flag, f"--tcrv-target-artifact-bundle-output-dir={tmp_path / 'missing'}"], p)
    assert r.returncode != 0 and "does not exist" in r.stderr
    # a tampered plan reaches no file
    out = tmp_path / "b"
    out.mkdir()
    bad = p.replace("tcrv_cuda.element_type=f32", "tcrv_cuda.element_type=f16", 1)
    r = run([TRANSLATE, "-", flag, f"--tcrv-target-artifact-bundle-output-dir={out}"], bad)
    assert r.returncode != 0 and "stale emission plan" in r.stderr and os.listdir(out) == []
    # without providers there is no bundle, no exporter and no translate route
    r = run([TRANSLATE, "-", "--tcrv-disable-builtin-plugins", flag, f"--tcrv-target-artifact-bundle-output-dir={out}"], p)
    assert r.returncode != 0 and 'no provider named "cuda-plugin"' in r.stderr and os.listdir(out) == []
    r = run([TRANSLATE, "-", "--tcrv-disable-builtin-plugins", "--tcrv-cuda-launch-to-cpp"], p)
    assert r.returncode != 0 and "unknown option '--tcrv-cuda-launch-to-cpp'" in r.stderr
    r = run([TRANSLATE, "-", "--tcrv-export-target-artifact", "--tcrv-export-emission-manifest"], p)
    assert r.returncode != 0 and "more than one translation" in r.stderr


# ---- abstract contraction request (tcrv_rvv.quant_contraction) -> provider picks the kernel

LOWER = "--tcrv-cuda-lower-quant-contraction"


def test_quant_contraction_decode_lowers_to_block_dot_with_audit():
    src = fixture("cuda-quant-contraction-q4-0.mlir")
    lowered = plan(src, [LOWER])
    assert "tcrv_rvv.quant_contraction" not in lowered
    assert "tcrv_rvv.q4_0_q8_0_block_dot %vx, %vy, %s, %n, %vl" in lowered  # the column count is dropped
    for needle in ('kind = "ggml_q4_0_q8_0_block_dot"', 'tcrv_cuda.contraction_algorithm = "decode-gemv-bulk-copy"',
                   'tcrv_cuda.path_selection_reason = "streaming-kept-q4_0-decode-hbm-bound"',
                   'tcrv_cuda.weight_layout_contract = "plain"', "weight_block_stride = 18"):
        assert needle in lowered, needle
    for gone in ("m_regime", "weight_layout =", "min_vlen", 'quant = "q4_0"'):
        assert gone not in lowered, gone
    h = header(plan(src, [LOWER, *PLAN_PASSES]))
    assert h.returncode == 0, h.stderr
    assert "void tcrv_emitc_ggml_vec_dot_q4_0_q8_0_kernel_ggml_vec_dot_q4_0_q8_0(size_t n, float *s, size_t bs" in h.stdout
    # lowering is idempotent; an unlowered request has no kernel
    assert plan(lowered, [LOWER]) == lowered
    r = run([OPT, "-", *PLAN_PASSES], src)
    assert r.returncode != 0 and "no kernel for op 'tcrv_rvv.quant_contraction'" in r.stderr


def test_quant_contraction_selection_matrix():
    src = fixture("cuda-quant-contraction-q4-0.mlir")
    prefill = plan(src.replace('m_regime = "decode"', 'm_regime = "prefill"'), [LOWER])
    assert 'tcrv_cuda.contraction_algorithm = "prefill-gemm-tcgen05-i8"' in prefill
    assert 'tcrv_cuda.path_selection_reason = "tensor-core-kept-q4_0-prefill"' in prefill
    assert 'tcrv_cuda.weight_layout_contract = "planar-int8-fp32-scales"' in prefill
    q8 = (src.replace('quant = "q4_0"', 'quant = "q8_0"').replace("weight_block_stride = 18", "weight_block_stride = 34")
          .replace(", activation_high_byte_offset = 16 : i64", ""))
    low = plan(q8, [LOWER])
    assert "tcrv_rvv.q8_0_q8_0_block_dot" in low and "streaming-kept-q8_0-decode-hbm-bound" in low
    low = plan(q8.replace('m_regime = "decode"', 'm_regime = "prefill"'), [LOWER])
    assert "streaming-decline-q8_0-no-tensor-core-kernel" in low and 'weight_layout_contract = "plain"' in low


@pytest.mark.parametrize("old,new,message", [
    ('weight_layout = "plain"', 'weight_layout = "x16"', "takes plain weights"),
    ('m_regime = "decode"', 'm_regime = "training"', "m_regime must be"),
    ('quant = "q4_0"', 'quant = "q4_K"', "unsupported quant"),
    ("weight_block_stride = 18", "weight_block_stride = 34", "needs weight_block_stride = 18"),
    ("%n, %bs, %vl {quant", "%n, %vl {quant", "takes weight, activation, output, n, nc"),
])
def test_quant_contraction_negatives(old, new, message):
    src = fixture("cuda-quant-contraction-q4-0.mlir")
    assert old in src
    r = run([OPT, "-", LOWER], src.replace(old, new))
    assert r.returncode != 0 and message in r.stderr, r.stderr
