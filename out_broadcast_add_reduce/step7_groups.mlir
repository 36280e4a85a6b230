// Config 3: out[m] = sum_n (b[m] + x[m, n]) on f32, f32 accumulation from zero.
#vec = affine_map<(d0, d1) -> (d0)>
#mat = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @broadcast_add_reduce(%b: tensor<?xf32>, %x: tensor<?x?xf32>) -> tensor<?xf32> attributes {afir.fused_group = "row_reduce", ascendc.kernel_kind = "vec", afir.cuda_kernel_class = "row_reduce", afir.cuda_launch = "{\"format\":\"afir-cuda-launch\",\"version\":1,\"kernel\":\"broadcast_add_reduce\",\"kernel_class\":\"row_reduce\",\"arch\":\"sm_100a\",\"dtype\":\"f32\",\"num_inputs\":2,\"num_outputs\":1,\"tiling\":[{\"name\":\"CTA_THREADS\",\"type\":\"int64\"},{\"name\":\"TEAM_LANES\",\"type\":\"int64\"},{\"name\":\"SPLIT_N\",\"type\":\"int64\"},{\"name\":\"BULK_COPY\",\"type\":\"int64\"},{\"name\":\"STREAM_STAGES\",\"type\":\"int64\"},{\"name\":\"STREAM_CHUNK\",\"type\":\"int64\"},{\"name\":\"dim_arg0_0\",\"type\":\"int64\"},{\"name\":\"dim_arg1_0\",\"type\":\"int64\"},{\"name\":\"dim_arg1_1\",\"type\":\"int64\"}],\"launch\":{\"cta_threads\":\"CTA_THREADS\",\"team_lanes\":\"TEAM_LANES\",\"split_cols\":\"SPLIT_N\",\"bulk_copy\":\"BULK_COPY\",\"stream_stages\":\"STREAM_STAGES\",\"stream_chunk_bytes\":\"STREAM_CHUNK\"},\"domain\":[\"dim_arg1_0\",\"dim_arg1_1\"],\"loads\":[{\"arg\":0,\"dtype\":\"f32\",\"shape\":[\"dim_arg0_0\"],\"map\":[0]},{\"arg\":1,\"dtype\":\"f32\",\"shape\":[\"dim_arg1_0\",\"dim_arg1_1\"],\"map\":[0,1]}],\"store\":{\"arg\":2,\"dtype\":\"f32\",\"shape\":[\"dim_arg1_0\"],\"map\":[0]},\"body\":[{\"op\":\"addf\",\"a\":\"v0\",\"b\":\"v1\"}]}"} {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %zero = arith.constant 0.0 : f32
    %m = tensor.dim %x, %c0 : tensor<?x?xf32>
    %n = tensor.dim %x, %c1 : tensor<?x?xf32>
    %e = tensor.empty(%m, %n) : tensor<?x?xf32>
    
    %acc0 = tensor.empty(%m) : tensor<?xf32>
    %init = linalg.fill ins(%zero : f32) outs(%acc0 : tensor<?xf32>) -> tensor<?xf32>
    %out = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0)>, affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>], iterator_types = ["parallel", "reduction"]}
        ins(%b, %x : tensor<?xf32>, tensor<?x?xf32>) outs(%init : tensor<?xf32>) {
    ^bb0(%in0: f32, %in1: f32, %acc: f32):
      %f0 = arith.addf %in0, %in1 : f32
      %sum = arith.addf %acc, %f0 : f32
      linalg.yield %sum : f32
    } -> tensor<?xf32>
    return %out : tensor<?xf32>
  }
}
