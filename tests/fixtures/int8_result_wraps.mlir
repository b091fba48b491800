module @jit_f {
  func.func public @main(%arg0: tensor<5x7xi8>, %arg1: tensor<7x3xi8>) -> tensor<5x3xi8> {
    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0] : (tensor<5x7xi8>, tensor<7x3xi8>) -> tensor<5x3xi8>
    return %0 : tensor<5x3xi8>
  }
}
