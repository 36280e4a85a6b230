// An elementwise group with an operand read through a transposed view: out[n, m] = a[m, n] + b[n, m] on f16.
#t = affine_map<(d0, d1) -> (d1, d0)>
#id = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @transposed_add(%a: tensor<?x?xf16>, %b: tensor<?x?xf16>) -> tensor<?x?xf16> {
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
