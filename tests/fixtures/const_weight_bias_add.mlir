module @jit_f {
  func.func public @main(%arg0: tensor<8x4xf32>, %arg1: tensor<3xf32>) -> tensor<8x3xf32> {
    %cst = stablehlo.constant dense<[[1, -2, 3], [4, 5, -6], [-7, 8, 9], [10, -11, 12]]> : tensor<4x3xi8>
    %cst_0 = stablehlo.constant dense<[5.000000e-01, 2.500000e-01, 2.000000e+00]> : tensor<3xf32>
    %0 = stablehlo.convert %cst : (tensor<4x3xi8>) -> tensor<4x3xf32>
    %1 = stablehlo.broadcast_in_dim %cst_0, dims = [1] : (tensor<3xf32>) -> tensor<4x3xf32>
    %2 = stablehlo.multiply %0, %1 : tensor<4x3xf32>
    %3 = stablehlo.dot_general %arg0, %2, contracting_dims = [1] x [0] : (tensor<8x4xf32>, tensor<4x3xf32>) -> tensor<8x3xf32>
    %4 = stablehlo.broadcast_in_dim %arg1, dims = [1] : (tensor<3xf32>) -> tensor<8x3xf32>
    %5 = stablehlo.add %3, %4 : tensor<8x3xf32>
    return %5 : tensor<8x3xf32>
  }
}
