module @jit_f {
  func.func public @main(%arg0: tensor<4x8x256xf32>, %arg1: tensor<256x128xi8>, %arg2: tensor<128xf32>) -> tensor<4x8x128xf32> {
    %0 = stablehlo.reshape %arg2 : (tensor<128xf32>) -> tensor<1x128xf32>
    %1 = stablehlo.broadcast_in_dim %0, dims = [0, 1] : (tensor<1x128xf32>) -> tensor<256x128xf32>
    %2 = stablehlo.convert %arg1 : (tensor<256x128xi8>) -> tensor<256x128xf32>
    %3 = stablehlo.multiply %1, %2 : tensor<256x128xf32>
    %4 = stablehlo.dot_general %arg0, %3, contracting_dims = [2] x [0] : (tensor<4x8x256xf32>, tensor<256x128xf32>) -> tensor<4x8x128xf32>
    return %4 : tensor<4x8x128xf32>
  }
}
