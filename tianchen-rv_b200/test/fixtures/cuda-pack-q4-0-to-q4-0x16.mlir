// plain block_q4_0 -> block_q4_0x16 weight repack body for the CUDA provider (envelope of the
// reference's test/Conversion/RVV/rvv-to-emitc-pack-q4-0-to-q4-0x16.mlir).
module {
  tcrv.exec.kernel @ggml_pack_q4_0_to_q4_0x16_kernel {
    tcrv.exec.capability @cuda {id = "cuda.sm_100a", kind = "accelerator", status = "available"}
    tcrv.exec.variant @ggml_pack_q4_0_to_q4_0x16 attributes {origin = "cuda-plugin", requires = [@cuda], tcrv_rvv.policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>} {
      %nblocks = tcrv_rvv.runtime_abi_value {c_name = "nblocks", c_type = "size_t", ownership = "target-export-abi-owned", purpose = "nblocks", role = "runtime-element-count"} : index
      %src = tcrv_rvv.runtime_abi_value {c_name = "src", c_type = "const uint8_t *", ownership = "target-export-abi-owned", purpose = "q4-plain-src", role = "lhs-input-buffer"} : !tcrv_rvv.runtime_abi_value
      %dst = tcrv_rvv.runtime_abi_value {c_name = "dst", c_type = "uint8_t *", ownership = "target-export-abi-owned", purpose = "q4x16-dst", role = "output-buffer"} : !tcrv_rvv.runtime_abi_value
      %vl = tcrv_rvv.setvl %nblocks {lmul = "m1", policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>, sew = 8 : i64} : index -> !tcrv_rvv.vl
      tcrv_rvv.with_vl %vl attributes {cuda_construction_protocol = "extension-family-construction-protocol.v1", lmul = "m1", origin = "cuda-plugin", policy = #tcrv_rvv.policy<tail = agnostic, mask = agnostic>, required_capabilities = [@cuda], selected_path_role = "direct call", selected_variant = @ggml_pack_q4_0_to_q4_0x16, sew = 8 : i64, source_kernel = "ggml_pack_q4_0_to_q4_0x16_kernel", status = "selected-lowering-boundary"} {
        %p = tcrv_rvv.pack_q4_0_to_q4_0x16 %src, %dst, %nblocks, %vl {kind = "ggml_pack_q4_0_to_q4_0x16", qk = 32 : i64, src_block_stride = 18 : i64, dst_block_stride = 288 : i64, src_quant_byte_offset = 2 : i64, dst_quant_byte_offset = 32 : i64, weight_interleave = 16 : i64, xor_mask = 136 : i64} : !tcrv_rvv.runtime_abi_value, !tcrv_rvv.runtime_abi_value, index, !tcrv_rvv.vl -> !tcrv_rvv.vector<i8, "m1">
      } : !tcrv_rvv.vl
    }
  }
}
