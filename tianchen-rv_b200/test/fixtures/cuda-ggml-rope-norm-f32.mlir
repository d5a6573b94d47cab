// ggml_rope_norm_f32 body for the CUDA provider (envelope of the reference's
// test/Conversion/RVV/rvv-to-emitc-ggml-rope-norm-f32.mlir).
module {
  tcrv.exec.kernel @ggml_rope_norm_f32_kernel {
    tcrv.exec.capability @cuda {id = "cuda.sm_100a", kind = "accelerator", status = "available"}
    tcrv.exec.variant @ggml_rope_norm_f32 attributes {origin = "cuda-plugin", requires = [@cuda], tcrv_rvv.policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>} {
      %n = tcrv_rvv.runtime_abi_value {c_name = "n_dims", c_type = "size_t", ownership = "target-export-abi-owned", purpose = "n", role = "runtime-element-count"} : index
      %x = tcrv_rvv.runtime_abi_value {c_name = "x", c_type = "const float *", ownership = "target-export-abi-owned", purpose = "in", role = "lhs-input-buffer"} : !tcrv_rvv.runtime_abi_value
      %y = tcrv_rvv.runtime_abi_value {c_name = "y", c_type = "float *", ownership = "target-export-abi-owned", purpose = "out", role = "output-buffer"} : !tcrv_rvv.runtime_abi_value
      %tb = tcrv_rvv.runtime_abi_value {c_name = "theta_base", c_type = "float", ownership = "target-export-abi-owned", purpose = "scale", role = "dequant-scale-value"} : !tcrv_rvv.runtime_abi_value
      %ts = tcrv_rvv.runtime_abi_value {c_name = "theta_scale", c_type = "float", ownership = "target-export-abi-owned", purpose = "scale", role = "dequant-scale-value"} : !tcrv_rvv.runtime_abi_value
      %vl = tcrv_rvv.setvl %n {lmul = "m1", policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>, sew = 32 : i64} : index -> !tcrv_rvv.vl
      tcrv_rvv.with_vl %vl attributes {cuda_construction_protocol = "extension-family-construction-protocol.v1", lmul = "m1", origin = "cuda-plugin", policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>, required_capabilities = [@cuda], selected_path_role = "direct call", selected_variant = @ggml_rope_norm_f32, sew = 32 : i64, source_kernel = "ggml_rope_norm_f32_kernel", status = "selected-lowering-boundary"} {
        %rot = tcrv_rvv.ggml_rope_norm_f32 %x, %y, %tb, %ts, %n, %vl {kind = "ggml_rope_norm_f32"} : !tcrv_rvv.runtime_abi_value, !tcrv_rvv.runtime_abi_value, !tcrv_rvv.runtime_abi_value, !tcrv_rvv.runtime_abi_value, index, !tcrv_rvv.vl -> !tcrv_rvv.vector<f32, "m1">
      } : !tcrv_rvv.vl
    }
  }
}
