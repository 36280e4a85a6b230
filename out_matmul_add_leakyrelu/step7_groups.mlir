// Config 5: out = max(x, 0.01 x), x = A . B + bias[n]; bf16 operands, f32 accumulation and epilogue, bf16 result.
#bias = affine_map<(d0, d1) -> (d1)>
#full = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @matmul_add_leakyrelu(%a: tensor<?x?xbf16>, %b: tensor<?x?xbf16>, %bias: tensor<?xbf16>) -> tensor<?x?xbf16> attributes {afir.fused_group = "matmul", ascendc.kernel_kind = "mix", abi_matmul_epilogue_kind = "BiasAddLeakyRelu", abi_matmul_has_bias = true, abi_matmul_layout_a = "ND", abi_matmul_layout_b = "ND", abi_matmul_layout_c = "ND", abi_matmul_op_kind = "matmul", abi_matmul_trans_a = false, abi_matmul_trans_b = false, afir.cuda_kernel_class = "matmul", afir.cuda_launch = "{\"format\":\"afir-cuda-launch\",\"version\":1,\"kernel\":\"matmul_add_leakyrelu\",\"kernel_class\":\"matmul\",\"arch\":\"sm_100a\",\"dtype\":\"bf16\",\"num_inputs\":3,\"num_outputs\":1,\"tiling\":[{\"name\":\"STAGES\",\"type\":\"int64\"},{\"name\":\"dim_arg0_0\",\"type\":\"int64\"},{\"name\":\"dim_arg0_1\",\"type\":\"int64\"},{\"name\":\"dim_arg1_1\",\"type\":\"int64\"}],\"launch\":{\"stages\":\"STAGES\"},\"matmul\":{\"a\":0,\"b\":1,\"bias\":2,\"out\":3,\"in_dtype\":\"bf16\",\"out_dtype\":\"bf16\",\"bias_dtype\":\"bf16\",\"epilogue\":\"BiasAddLeakyRelu\",\"alpha\":0.01,\"m\":\"dim_arg0_0\",\"n\":\"dim_arg1_1\",\"k\":\"dim_arg0_1\"}}"} {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %zero = arith.constant 0.0 : f32
    %alpha = arith.constant 1.0e-2 : f32
    %m = tensor.dim %a, %c0 : tensor<?x?xbf16>
    %n = tensor.dim %b, %c1 : tensor<?x?xbf16>
    %acc0 = tensor.empty(%m, %n) : tensor<?x?xf32>
    %init = linalg.fill ins(%zero : f32) outs(%acc0 : tensor<?x?xf32>) -> tensor<?x?xf32>
    %c = linalg.matmul ins(%a, %b : tensor<?x?xbf16>, tensor<?x?xbf16>) outs(%init : tensor<?x?xf32>) -> tensor<?x?xf32>
    %e = tensor.empty(%m, %n) : tensor<?x?xbf16>
    %r = linalg.generic {indexing_maps = [#full, #bias, #full], iterator_types = ["parallel", "parallel"]}
        ins(%c, %bias : tensor<?x?xf32>, tensor<?xbf16>) outs(%e : tensor<?x?xbf16>) {
    ^bb0(%cv: f32, %bv: bf16, %o: bf16):
      %bf = arith.extf %bv : bf16 to f32
      %x = arith.addf %cv, %bf : f32
      %s = arith.mulf %x, %alpha : f32
      %y = arith.maximumf %x, %s : f32
      %t = arith.truncf %y : f32 to bf16
      linalg.yield %t : bf16
    } -> tensor<?x?xbf16>
    return %r : tensor<?x?xbf16>
  }
}
