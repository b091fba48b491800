module @jit_f {
  func.func public @main(%arg0: tensor<16x256xbf16>, %arg1: tensor<128x256xi8>, %arg2: tensor<128xf32>) -> tensor<16x128xbf16> {
    %0 = stablehlo.convert %arg1 : (tensor<128x256xi8>) -> tensor<128x256xbf16>
    %1 = stablehlo.convert %arg2 : (tensor<128xf32>) -> tensor<128xbf16>
    %2 = stablehlo.broadcast_in_dim %1, dims = [0] : (tensor<128xbf16>) -> tensor<128x256xbf16>
    %3 = stablehlo.multiply %0, %2 : tensor<128x256xbf16>
    %4 = stablehlo.dot_general %arg0, %3, contracting_dims = [1] x [1] : (tensor<16x256xbf16>, tensor<128x256xbf16>) -> tensor<16x128xbf16>
    return %4 : tensor<16x128xbf16>
  }
}
