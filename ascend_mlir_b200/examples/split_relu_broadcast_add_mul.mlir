// Config 2: x f16 [B, R, 2C] split on the last axis into h0, h1; out = (relu(h0) + bias[r]) * h1.
#full = affine_map<(d0, d1, d2) -> (d0, d1, d2)>
#rows = affine_map<(d0, d1, d2) -> (d1)>
module {
  func.func @split_relu_broadcast_add_mul(%x: tensor<?x?x?xf16>, %bias: tensor<?xf16>) -> tensor<?x?x?xf16> {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %zero = arith.constant 0.0 : f16
    %b = tensor.dim %x, %c0 : tensor<?x?x?xf16>
    %r = tensor.dim %x, %c1 : tensor<?x?x?xf16>
    %c = tensor.dim %bias, %c0 : tensor<?xf16>
    %h0 = tensor.extract_slice %x[0, 0, 0][%b, %r, %c][1, 1, 1] : tensor<?x?x?xf16> to tensor<?x?x?xf16>
    %h1 = tensor.extract_slice %x[0, 0, %c][%b, %r, %c][1, 1, 1] : tensor<?x?x?xf16> to tensor<?x?x?xf16>
    %e0 = tensor.empty(%b, %r, %c) : tensor<?x?x?xf16>
    %t = linalg.generic {indexing_maps = [#full, #rows, #full], iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%h0, %bias : tensor<?x?x?xf16>, tensor<?xf16>) outs(%e0 : tensor<?x?x?xf16>) {
    ^bb0(%in: f16, %bv: f16, %o: f16):
      %m = arith.maximumf %in, %zero : f16
      %s = arith.addf %m, %bv : f16
      linalg.yield %s : f16
    } -> tensor<?x?x?xf16>
    %e1 = tensor.empty(%b, %r, %c) : tensor<?x?x?xf16>
    %out = linalg.generic {indexing_maps = [#full, #full, #full], iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%t, %h1 : tensor<?x?x?xf16>, tensor<?x?x?xf16>) outs(%e1 : tensor<?x?x?xf16>) {
    ^bb0(%u: f16, %v: f16, %o: f16):
      %p = arith.mulf %u, %v : f16
      linalg.yield %p : f16
    } -> tensor<?x?x?xf16>
    return %out : tensor<?x?x?xf16>
  }
}
