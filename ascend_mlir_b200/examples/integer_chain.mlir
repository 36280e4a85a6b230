// Integer elementwise group: out = (a + b[n]) * a on i16, two's-complement wrap-around (the AFIR binary ops admit
// i16 and i32 element types).
module {
  func.func @integer_chain(%a: tensor<333x1000xi16>, %b: tensor<1000xi16>) -> tensor<333x1000xi16> {
    %s = afir.add %a, %b : (tensor<333x1000xi16>, tensor<1000xi16>) -> tensor<333x1000xi16>
    %p = afir.mul %s, %a : (tensor<333x1000xi16>, tensor<333x1000xi16>) -> tensor<333x1000xi16>
    return %p : tensor<333x1000xi16>
  }
}
