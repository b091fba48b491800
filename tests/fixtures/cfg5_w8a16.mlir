module @jit_f {
  func.func public @main(%arg0: tensor<4096x8192xbf16>, %arg1: tensor<8192x1024xi8>, %arg2: tensor<1024xf32>) -> tensor<4096x1024xbf16> {
    %0 = stablehlo.convert %arg1 : (tensor<8192x1024xi8>) -> tensor<8192x1024xbf16>
    %1 = stablehlo.convert %arg2 : (tensor<1024xf32>) -> tensor<1024xbf16>
    %2 = stablehlo.broadcast_in_dim %1, dims = [1] : (tensor<1024xbf16>) -> tensor<8192x1024xbf16>
    %3 = stablehlo.multiply %0, %2 : tensor<8192x1024xbf16>
    %4 = stablehlo.dot_general %arg0, %3, contracting_dims = [1] x [0] : (tensor<4096x8192xbf16>, tensor<8192x1024xbf16>) -> tensor<4096x1024xbf16>
    return %4 : tensor<4096x1024xbf16>
  }
}
