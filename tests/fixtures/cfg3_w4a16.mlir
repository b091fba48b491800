module @jit_f attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<4x4096xbf16>, %arg1: tensor<2048x14336xui8>, %arg2: tensor<32x14336xbf16>, %arg3: tensor<32x14336xui4>) -> (tensor<4x14336xbf16> {jax.result_info = "result"}) {
    %c = stablehlo.constant dense<15> : tensor<ui8>
    %0 = stablehlo.broadcast_in_dim %c, dims = [] : (tensor<ui8>) -> tensor<2048x14336xui8>
    %1 = stablehlo.and %arg1, %0 : tensor<2048x14336xui8>
    %c_0 = stablehlo.constant dense<4> : tensor<ui8>
    %2 = stablehlo.broadcast_in_dim %c_0, dims = [] : (tensor<ui8>) -> tensor<2048x14336xui8>
    %3 = stablehlo.shift_right_logical %arg1, %2 : tensor<2048x14336xui8>
    %4 = stablehlo.broadcast_in_dim %1, dims = [0, 2] : (tensor<2048x14336xui8>) -> tensor<2048x1x14336xui8>
    %5 = stablehlo.broadcast_in_dim %3, dims = [0, 2] : (tensor<2048x14336xui8>) -> tensor<2048x1x14336xui8>
    %6 = stablehlo.concatenate %4, %5, dim = 1 : (tensor<2048x1x14336xui8>, tensor<2048x1x14336xui8>) -> tensor<2048x2x14336xui8>
    %7 = stablehlo.reshape %6 : (tensor<2048x2x14336xui8>) -> tensor<4096x14336xui8>
    %8 = stablehlo.convert %7 : (tensor<4096x14336xui8>) -> tensor<4096x14336xbf16>
    %9 = stablehlo.reshape %8 : (tensor<4096x14336xbf16>) -> tensor<32x128x14336xbf16>
    %10 = stablehlo.convert %arg3 : (tensor<32x14336xui4>) -> tensor<32x14336xbf16>
    %11 = stablehlo.broadcast_in_dim %10, dims = [0, 2] : (tensor<32x14336xbf16>) -> tensor<32x128x14336xbf16>
    %12 = stablehlo.subtract %9, %11 : tensor<32x128x14336xbf16>
    %13 = stablehlo.broadcast_in_dim %arg2, dims = [0, 2] : (tensor<32x14336xbf16>) -> tensor<32x128x14336xbf16>
    %14 = stablehlo.multiply %12, %13 : tensor<32x128x14336xbf16>
    %15 = stablehlo.reshape %14 : (tensor<32x128x14336xbf16>) -> tensor<4096x14336xbf16>
    %16 = stablehlo.dot_general %arg0, %15, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<4x4096xbf16>, tensor<4096x14336xbf16>) -> tensor<4x14336xbf16>
    return %16 : tensor<4x14336xbf16>
  }
}
