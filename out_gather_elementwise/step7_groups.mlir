// Config 4: out[i, :] = table[idx[i], :] * scale + resid[i, :] on bf16, i32 indices (row gather).
#rowidx = affine_map<(d0, d1) -> (d0)>
#cols = affine_map<(d0, d1) -> (d1)>
#full = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @gather_elementwise(%table: tensor<?x?xbf16>, %idx: tensor<?xi32>, %scale: tensor<?xbf16>, %resid: tensor<?x?xbf16>) -> tensor<?x?xbf16> attributes {afir.fused_group = "gather", ascendc.kernel_kind = "vec", afir.cuda_kernel_class = "gather", afir.cuda_launch = "{\"format\":\"afir-cuda-launch\",\"version\":1,\"kernel\":\"gather_elementwise\",\"kernel_class\":\"gather\",\"arch\":\"sm_100a\",\"dtype\":\"bf16\",\"num_inputs\":4,\"num_outputs\":1,\"tiling\":[{\"name\":\"CTA_THREADS\",\"type\":\"int64\"},{\"name\":\"UNROLL\",\"type\":\"int64\"},{\"name\":\"BULK_COPY\",\"type\":\"int64\"},{\"name\":\"STREAM_STAGES\",\"type\":\"int64\"},{\"name\":\"STREAM_ROWS\",\"type\":\"int64\"},{\"name\":\"STREAM_WARPS\",\"type\":\"int64\"},{\"name\":\"dim_arg0_0\",\"type\":\"int64\"},{\"name\":\"dim_arg0_1\",\"type\":\"int64\"},{\"name\":\"dim_arg1_0\",\"type\":\"int64\"},{\"name\":\"dim_arg2_0\",\"type\":\"int64\"},{\"name\":\"dim_arg3_0\",\"type\":\"int64\"},{\"name\":\"dim_arg3_1\",\"type\":\"int64\"}],\"launch\":{\"cta_threads\":\"CTA_THREADS\",\"unroll\":\"UNROLL\",\"bulk_copy\":\"BULK_COPY\",\"stream_stages\":\"STREAM_STAGES\",\"stream_rows\":\"STREAM_ROWS\",\"stream_warps\":\"STREAM_WARPS\"},\"domain\":[\"dim_arg1_0\",\"dim_arg0_1\"],\"loads\":[{\"arg\":0,\"dtype\":\"bf16\",\"shape\":[\"dim_arg0_0\",\"dim_arg0_1\"]},{\"arg\":2,\"dtype\":\"bf16\",\"shape\":[\"dim_arg2_0\"],\"map\":[1]},{\"arg\":3,\"dtype\":\"bf16\",\"shape\":[\"dim_arg3_0\",\"dim_arg3_1\"],\"map\":[0,1]}],\"store\":{\"arg\":4,\"dtype\":\"bf16\",\"shape\":[\"dim_arg1_0\",\"dim_arg0_1\"],\"map\":[0,1]},\"body\":[{\"op\":\"mulf\",\"a\":\"v0\",\"b\":\"v1\"},{\"op\":\"addf\",\"a\":\"%0\",\"b\":\"v2\"}],\"gather\":{\"axis\":0,\"indices\":{\"arg\":1,\"dtype\":\"i32\",\"shape\":[\"dim_arg1_0\"]}}}"} {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %rows = tensor.dim %idx, %c0 : tensor<?xi32>
    %width = tensor.dim %table, %c1 : tensor<?x?xbf16>
    %e0 = tensor.empty(%rows, %width) : tensor<?x?xbf16>
    
    %e1 = tensor.empty(%rows, %width) : tensor<?x?xbf16>
    %out = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0)>, affine_map<(d0, d1) -> (d1)>, affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>], iterator_types = ["parallel", "parallel"], embedding_dim = 0 : i64}
        ins(%idx, %scale, %resid : tensor<?xi32>, tensor<?xbf16>, tensor<?x?xbf16>) outs(%e1 : tensor<?x?xbf16>) {
    ^bb0(%idx: i32, %in1: bf16, %in2: bf16, %acc: bf16):
      %pos = linalg.index 1 : index
      %picked = arith.index_cast %idx : i32 to index
      %gathered = tensor.extract %table[%picked, %pos] : tensor<?x?xbf16>
      %f0 = arith.mulf %gathered, %in1 : bf16
      %f1 = arith.addf %f0, %in2 : bf16
      linalg.yield %f1 : bf16
    } -> tensor<?x?xbf16>
    return %out : tensor<?x?xbf16>
  }
}
