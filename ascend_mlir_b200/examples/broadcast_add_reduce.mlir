// Config 3: out[m] = sum_n (b[m] + x[m, n]) on f32, f32 accumulation from zero.
#vec = affine_map<(d0, d1) -> (d0)>
#mat = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @broadcast_add_reduce(%b: tensor<?xf32>, %x: tensor<?x?xf32>) -> tensor<?xf32> {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %zero = arith.constant 0.0 : f32
    %m = tensor.dim %x, %c0 : tensor<?x?xf32>
    %n = tensor.dim %x, %c1 : tensor<?x?xf32>
    %e = tensor.empty(%m, %n) : tensor<?x?xf32>
    %sum = linalg.generic {indexing_maps = [#vec, #mat, #mat], iterator_types = ["parallel", "parallel"]}
        ins(%b, %x : tensor<?xf32>, tensor<?x?xf32>) outs(%e : tensor<?x?xf32>) {
    ^bb0(%bv: f32, %xv: f32, %o: f32):
      %s = arith.addf %bv, %xv : f32
      linalg.yield %s : f32
    } -> tensor<?x?xf32>
    %acc0 = tensor.empty(%m) : tensor<?xf32>
    %init = linalg.fill ins(%zero : f32) outs(%acc0 : tensor<?xf32>) -> tensor<?xf32>
    %out = linalg.generic {indexing_maps = [#mat, #vec], iterator_types = ["parallel", "reduction"]}
        ins(%sum : tensor<?x?xf32>) outs(%init : tensor<?xf32>) {
    ^bb0(%v: f32, %acc: f32):
      %a = arith.addf %acc, %v : f32
      linalg.yield %a : f32
    } -> tensor<?xf32>
    return %out : tensor<?xf32>
  }
}
