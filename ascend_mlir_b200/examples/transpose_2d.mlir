// Standalone permutation group: out[c, r] = in[r, c] on f16.
#in = affine_map<(d0, d1) -> (d1, d0)>
#out = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @transpose_2d(%x: tensor<?x?xf16>) -> tensor<?x?xf16> {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %r = tensor.dim %x, %c0 : tensor<?x?xf16>
    %c = tensor.dim %x, %c1 : tensor<?x?xf16>
    %e = tensor.empty(%c, %r) : tensor<?x?xf16>
    %t = linalg.generic {indexing_maps = [#in, #out], iterator_types = ["parallel", "parallel"]}
        ins(%x : tensor<?x?xf16>) outs(%e : tensor<?x?xf16>) {
    ^bb0(%v: f16, %o: f16):
      linalg.yield %v : f16
    } -> tensor<?x?xf16>
    return %t : tensor<?x?xf16>
  }
}
