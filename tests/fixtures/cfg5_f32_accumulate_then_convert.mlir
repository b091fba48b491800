module @jit_f {
  func.func public @main(%arg0: tensor<256x512xbf16>, %arg1: tensor<512x384xi8>, %arg2: tensor<384xf32>) -> tensor<256x384xbf16> {
    %0 = stablehlo.convert %arg1 : (tensor<512x384xi8>) -> tensor<512x384xbf16>
    %1 = stablehlo.convert %arg2 : (tensor<384xf32>) -> tensor<384xbf16>
    %2 = stablehlo.broadcast_in_dim %1, dims = [1] : (tensor<384xbf16>) -> tensor<512x384xbf16>
    %3 = stablehlo.multiply %0, %2 : tensor<512x384xbf16>
    %4 = stablehlo.dot_general %arg0, %3, contracting_dims = [1] x [0] : (tensor<256x512xbf16>, tensor<512x384xbf16>) -> tensor<256x384xf32>
    %5 = stablehlo.convert %4 : (tensor<256x384xf32>) -> tensor<256x384xbf16>
    return %5 : tensor<256x384xbf16>
  }
}
