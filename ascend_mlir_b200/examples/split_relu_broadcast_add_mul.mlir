// Config 2: x f16 [32, 1024, 2048] split on the last axis into h0, h1; out = (relu(h0) + bias[r]) * h1.
#full = affine_map<(d0, d1, d2) -> (d0, d1, d2)>
#rows = affine_map<(d0, d1, d2) -> (d1)>
module {
  func.func @split_relu_broadcast_add_mul(%x: tensor<32x1024x2048xf16>, %bias: tensor<1024xf16>) -> tensor<32x1024x1024xf16> {
    %zero = arith.constant 0.0 : f16
    %h0 = tensor.extract_slice %x[0, 0, 0][32, 1024, 1024][1, 1, 1] : tensor<32x1024x2048xf16> to tensor<32x1024x1024xf16>
    %h1 = tensor.extract_slice %x[0, 0, 1024][32, 1024, 1024][1, 1, 1] : tensor<32x1024x2048xf16> to tensor<32x1024x1024xf16>
    %e0 = tensor.empty() : tensor<32x1024x1024xf16>
    %t = linalg.generic {indexing_maps = [#full, #rows, #full], iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%h0, %bias : tensor<32x1024x1024xf16>, tensor<1024xf16>) outs(%e0 : tensor<32x1024x1024xf16>) {
    ^bb0(%in: f16, %bv: f16, %o: f16):
      %m = arith.maximumf %in, %zero : f16
      %s = arith.addf %m, %bv : f16
      linalg.yield %s : f16
    } -> tensor<32x1024x1024xf16>
    %e1 = tensor.empty() : tensor<32x1024x1024xf16>
    %out = linalg.generic {indexing_maps = [#full, #full, #full], iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%t, %h1 : tensor<32x1024x1024xf16>, tensor<32x1024x1024xf16>) outs(%e1 : tensor<32x1024x1024xf16>) {
    ^bb0(%u: f16, %v: f16, %o: f16):
      %p = arith.mulf %u, %v : f16
      linalg.yield %p : f16
    } -> tensor<32x1024x1024xf16>
    return %out : tensor<32x1024x1024xf16>
  }
}
