// Config 1: out = (a + b) * b on f32 [4096, 4096], written with the AFIR elementwise ops.
module {
  func.func @elementwise_chain(%a: tensor<4096x4096xf32>, %b: tensor<4096x4096xf32>) -> tensor<4096x4096xf32> {
    %s = afir.add %a, %b : (tensor<4096x4096xf32>, tensor<4096x4096xf32>) -> tensor<4096x4096xf32>
    %p = afir.mul %s, %b : (tensor<4096x4096xf32>, tensor<4096x4096xf32>) -> tensor<4096x4096xf32>
    return %p : tensor<4096x4096xf32>
  }
}
