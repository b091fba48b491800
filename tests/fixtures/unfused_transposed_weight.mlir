module @jit_f {
  func.func public @main(%arg0: tensor<16x256xf32>, %arg1: tensor<128x256xi8>, %arg2: tensor<128xf32>) -> tensor<16x128xf32> {
    %0 = stablehlo.convert %arg1 : (tensor<128x256xi8>) -> tensor<128x256xf32>
    %1 = stablehlo.broadcast_in_dim %arg2, dims = [0] : (tensor<128xf32>) -> tensor<128x256xf32>
    %2 = stablehlo.multiply %0, %1 : tensor<128x256xf32>
    %3 = stablehlo.transpose %2, dims = [1, 0] : (tensor<128x256xf32>) -> tensor<256x128xf32>
    %4 = stablehlo.dot_general %arg0, %3, contracting_dims = [1] x [0] : (tensor<16x256xf32>, tensor<256x128xf32>) -> tensor<16x128xf32>
    return %4 : tensor<16x128xf32>
  }
}
