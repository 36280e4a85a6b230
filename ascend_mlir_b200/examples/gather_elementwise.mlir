// Config 4: out[i, :] = table[idx[i], :] * scale + resid[i, :] on bf16, i32 indices (row gather).
#rowidx = affine_map<(d0, d1) -> (d0)>
#cols = affine_map<(d0, d1) -> (d1)>
#full = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @gather_elementwise(%table: tensor<?x?xbf16>, %idx: tensor<?xi32>, %scale: tensor<?xbf16>, %resid: tensor<?x?xbf16>) -> tensor<?x?xbf16> {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %rows = tensor.dim %idx, %c0 : tensor<?xi32>
    %width = tensor.dim %table, %c1 : tensor<?x?xbf16>
    %e0 = tensor.empty(%rows, %width) : tensor<?x?xbf16>
    %g = linalg.generic {indexing_maps = [#rowidx, #full], iterator_types = ["parallel", "parallel"]}
        ins(%idx : tensor<?xi32>) outs(%e0 : tensor<?x?xbf16>) {
    ^bb0(%i32: i32, %o: bf16):
      %j = linalg.index 1 : index
      %r = arith.index_cast %i32 : i32 to index
      %v = tensor.extract %table[%r, %j] : tensor<?x?xbf16>
      linalg.yield %v : bf16
    } -> tensor<?x?xbf16>
    %e1 = tensor.empty(%rows, %width) : tensor<?x?xbf16>
    %out = linalg.generic {indexing_maps = [#full, #cols, #full, #full], iterator_types = ["parallel", "parallel"]}
        ins(%g, %scale, %resid : tensor<?x?xbf16>, tensor<?xbf16>, tensor<?x?xbf16>) outs(%e1 : tensor<?x?xbf16>) {
    ^bb0(%gv: bf16, %sv: bf16, %rv: bf16, %o: bf16):
      %p = arith.mulf %gv, %sv : bf16
      %s = arith.addf %p, %rv : bf16
      linalg.yield %s : bf16
    } -> tensor<?x?xbf16>
    return %out : tensor<?x?xbf16>
  }
}
