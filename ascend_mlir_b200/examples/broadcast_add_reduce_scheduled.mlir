// Config 3 with a tiling schedule beside it, the form the reference keeps its strategies in: out[m] = sum_n (b[m] + x[m, n]).
// The schedule adds three index arguments to the kernel (rows per CTA group, rows per step, columns per step), tiles the
// row axis twice and the reduced axis once, and marks the outer row loop as the one spread over the machine.
// `afir-opt --transform-interpreter` records the schedule on the function; the sm_100a kernel is generated from the
// fused group as a whole, so no loop nest is materialised.
#vec = affine_map<(d0, d1) -> (d0)>
#mat = affine_map<(d0, d1) -> (d0, d1)>
module attributes {transform.with_named_sequence} {
  func.func @broadcast_add_reduce_scheduled(%b: tensor<?xf32>, %x: tensor<?x?xf32>) -> tensor<?xf32> {
    %c0 = arith.constant 0 : index
    %zero = arith.constant 0.0 : f32
    %m = tensor.dim %x, %c0 : tensor<?x?xf32>
    %acc0 = tensor.empty(%m) : tensor<?xf32>
    %init = linalg.fill ins(%zero : f32) outs(%acc0 : tensor<?xf32>) -> tensor<?xf32>
    %out = linalg.generic {indexing_maps = [#vec, #mat, #vec], iterator_types = ["parallel", "reduction"]}
        ins(%b, %x : tensor<?xf32>, tensor<?x?xf32>) outs(%init : tensor<?xf32>) {
    ^bb0(%bv: f32, %xv: f32, %acc: f32):
      %s = arith.addf %bv, %xv : f32
      %a = arith.addf %acc, %s : f32
      linalg.yield %a : f32
    } -> tensor<?xf32>
    return %out : tensor<?xf32>
  }

  transform.named_sequence @__transform_main(%root : !transform.any_op {transform.readonly}) {
    %func = transform.structured.match ops{["func.func"]} in %root : (!transform.any_op) -> !transform.any_op
    %with_args, %rows_per_group, %rows_per_step, %cols_per_step = transform.func.add_index_args %func, 3
        : (!transform.any_op) -> (!transform.any_op, !transform.any_op, !transform.any_op, !transform.any_op)
    %group = transform.structured.match ops{["linalg.generic"]} in %with_args : (!transform.any_op) -> !transform.any_op
    %inner, %row_loop = transform.structured.tile_using_for %group tile_sizes [%rows_per_group, 0]
        : (!transform.any_op, !transform.any_op) -> (!transform.any_op, !transform.any_op)
    %spread = transform.param.constant true -> !transform.any_param
    transform.annotate %row_loop "ascendc.parallel" = %spread : !transform.any_op, !transform.any_param
    %step, %step_rows, %step_cols = transform.structured.tile_using_for %inner tile_sizes [%rows_per_step, %cols_per_step]
        : (!transform.any_op, !transform.any_op, !transform.any_op) -> (!transform.any_op, !transform.any_op, !transform.any_op)
    %unit = transform.param.constant "AiCore.Vector" -> !transform.any_param
    transform.annotate %step "ascendc.unit" = %unit : !transform.any_op, !transform.any_param
    transform.yield
  }
}
