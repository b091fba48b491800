module @jit_f {
  func.func public @main(%arg0: tensor<32x1024xf32>, %arg1: tensor<1024x1024xi8>, %arg2: tensor<1024xf32>) -> (tensor<32x1024xf32>, tensor<1024x1024xf32>) {
    %0 = stablehlo.convert %arg1 : (tensor<1024x1024xi8>) -> tensor<1024x1024xf32>
    %1 = stablehlo.broadcast_in_dim %arg2, dims = [1] : (tensor<1024xf32>) -> tensor<1024x1024xf32>
    %2 = stablehlo.multiply %0, %1 : tensor<1024x1024xf32>
    %3 = stablehlo.dot_general %arg0, %2, contracting_dims = [1] x [0] : (tensor<32x1024xf32>, tensor<1024x1024xf32>) -> tensor<32x1024xf32>
    %4 = stablehlo.negate %2 : tensor<1024x1024xf32>
    return %3, %4 : tensor<32x1024xf32>, tensor<1024x1024xf32>
  }
}
