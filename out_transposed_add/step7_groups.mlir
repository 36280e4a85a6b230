// An elementwise group with an operand read through a transposed view: out[n, m] = a[m, n] + b[n, m] on f16.
#t = affine_map<(d0, d1) -> (d1, d0)>
#id = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @transposed_add(%a: tensor<?x?xf16>, %b: tensor<?x?xf16>) -> tensor<?x?xf16> attributes {afir.fused_group = "elementwise", ascendc.kernel_kind = "vec", afir.cuda_kernel_class = "elementwise", afir.cuda_launch = "{\"format\":\"afir-cuda-launch\",\"version\":1,\"kernel\":\"transposed_add\",\"kernel_class\":\"elementwise\",\"arch\":\"sm_100a\",\"dtype\":\"f16\",\"num_inputs\":2,\"num_outputs\":1,\"tiling\":[{\"name\":\"CTA_THREADS\",\"type\":\"int64\"},{\"name\":\"UNROLL\",\"type\":\"int64\"},{\"name\":\"dim_arg0_0\",\"type\":\"int64\"},{\"name\":\"dim_arg0_1\",\"type\":\"int64\"},{\"name\":\"dim_arg1_0\",\"type\":\"int64\"},{\"name\":\"dim_arg1_1\",\"type\":\"int64\"}],\"launch\":{\"cta_threads\":\"CTA_THREADS\",\"unroll\":\"UNROLL\"},\"domain\":[\"dim_arg1_0\",\"dim_arg1_1\"],\"loads\":[{\"arg\":0,\"dtype\":\"f16\",\"shape\":[\"dim_arg0_0\",\"dim_arg0_1\"],\"map\":[1,0]},{\"arg\":1,\"dtype\":\"f16\",\"shape\":[\"dim_arg1_0\",\"dim_arg1_1\"],\"map\":[0,1]}],\"store\":{\"arg\":2,\"dtype\":\"f16\",\"shape\":[\"dim_arg1_0\",\"dim_arg1_1\"],\"map\":[0,1]},\"body\":[{\"op\":\"addf\",\"a\":\"v0\",\"b\":\"v1\"}]}"} {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %n = tensor.dim %b, %c0 : tensor<?x?xf16>
    %m = tensor.dim %b, %c1 : tensor<?x?xf16>
    %e = tensor.empty(%n, %m) : tensor<?x?xf16>
    %r = linalg.generic {indexing_maps = [#t, #id, #id], iterator_types = ["parallel", "parallel"]}
        ins(%a, %b : tensor<?x?xf16>, tensor<?x?xf16>) outs(%e : tensor<?x?xf16>) {
    ^bb0(%x: f16, %y: f16, %o: f16):
      %s = arith.addf %x, %y : f16
      linalg.yield %s : f16
    } -> tensor<?x?xf16>
    return %r : tensor<?x?xf16>
  }
}
