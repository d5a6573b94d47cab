// ggml Q4_0 x Q8_0 GEMM tile (one weight row against activation_cols columns) for the CUDA provider
// (envelope of the reference's test/Conversion/RVV/rvv-to-emitc-q4-0-q8-0-gemm-tile.mlir; ABI order
// n, s, vx, vy, by; the column count is a compile-time attribute of the op).
module {
  tcrv.exec.kernel @ggml_q4_0_q8_0_gemm_tile_kernel {
    tcrv.exec.capability @cuda {id = "cuda.sm_100a", kind = "accelerator", status = "available"}
    tcrv.exec.variant @ggml_q4_0_q8_0_gemm_tile attributes {origin = "cuda-plugin", requires = [@cuda], tcrv_rvv.policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>} {
      %n = tcrv_rvv.runtime_abi_value {c_name = "n", c_type = "size_t", ownership = "target-export-abi-owned", purpose = "n", role = "runtime-element-count"} : index
      %s = tcrv_rvv.runtime_abi_value {c_name = "s", c_type = "float *", ownership = "target-export-abi-owned", purpose = "out", role = "output-buffer"} : !tcrv_rvv.runtime_abi_value
      %vx = tcrv_rvv.runtime_abi_value {c_name = "vx", c_type = "const uint8_t *", ownership = "target-export-abi-owned", purpose = "q4-weight", role = "lhs-input-buffer"} : !tcrv_rvv.runtime_abi_value
      %vy = tcrv_rvv.runtime_abi_value {c_name = "vy", c_type = "const uint8_t *", ownership = "target-export-abi-owned", purpose = "q8-act", role = "rhs-input-buffer"} : !tcrv_rvv.runtime_abi_value
      %by = tcrv_rvv.runtime_abi_value {c_name = "by", c_type = "size_t", ownership = "target-export-abi-owned", purpose = "by", role = "rhs-input-stride"} : index
      %vl = tcrv_rvv.setvl %n {lmul = "m1", policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>, sew = 32 : i64} : index -> !tcrv_rvv.vl
      tcrv_rvv.with_vl %vl attributes {cuda_construction_protocol = "extension-family-construction-protocol.v1", lmul = "m1", origin = "cuda-plugin", policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>, required_capabilities = [@cuda], selected_path_role = "direct call", selected_variant = @ggml_q4_0_q8_0_gemm_tile, sew = 32 : i64, source_kernel = "ggml_q4_0_q8_0_gemm_tile_kernel", status = "selected-lowering-boundary"} {
        %tile = tcrv_rvv.q4_0_q8_0_gemm_tile %vx, %vy, %by, %s, %n, %vl {kind = "ggml_q4_0_q8_0_gemm_tile", scale_model = "dual-fp16-per-block-d_x.d_y", qk = 32 : i64, weight_block_stride = 18 : i64, activation_block_stride = 34 : i64, quant_byte_offset = 2 : i64, activation_high_byte_offset = 16 : i64, activation_cols = 4 : i64} : !tcrv_rvv.runtime_abi_value, !tcrv_rvv.runtime_abi_value, index, !tcrv_rvv.runtime_abi_value, index, !tcrv_rvv.vl -> !tcrv_rvv.vector<i32, "m1">
      } : !tcrv_rvv.vl
    }
  }
}
