module @jit_f {
  func.func public @main(%arg0: tensor<32x256xf32>, %arg1: tensor<256x128xi8>, %arg2: tensor<128xf32>) -> tensor<32x128xf32> {
    %0 = stablehlo.convert %arg1 : (tensor<256x128xi8>) -> tensor<256x128xf32>
    %1 = stablehlo.broadcast_in_dim %arg2, dims = [1] : (tensor<128xf32>) -> tensor<256x128xf32>
    %2 = stablehlo.multiply %0, %1 : tensor<256x128xf32>
    %3 = stablehlo.dot %arg0, %2 : (tensor<32x256xf32>, tensor<256x128xf32>) -> tensor<32x128xf32>
    return %3 : tensor<32x128xf32>
  }
}
