module @jit_f attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<2048x4096xi8>, %arg1: tensor<4096x4096xi8>, %arg2: tensor<2048xf32>, %arg3: tensor<4096xf32>) -> (tensor<2048x4096xi32>, tensor<2048x4096xf32>) {
    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0] : (tensor<2048x4096xi8>, tensor<4096x4096xi8>) -> tensor<2048x4096xi32>
    %1 = stablehlo.convert %0 : (tensor<2048x4096xi32>) -> tensor<2048x4096xf32>
    %2 = stablehlo.broadcast_in_dim %arg2, dims = [0] : (tensor<2048xf32>) -> tensor<2048x1xf32>
    %3 = stablehlo.broadcast_in_dim %2, dims = [0, 1] : (tensor<2048x1xf32>) -> tensor<2048x4096xf32>
    %4 = stablehlo.multiply %1, %3 : tensor<2048x4096xf32>
    %5 = stablehlo.broadcast_in_dim %arg3, dims = [1] : (tensor<4096xf32>) -> tensor<1x4096xf32>
    %6 = stablehlo.broadcast_in_dim %5, dims = [0, 1] : (tensor<1x4096xf32>) -> tensor<2048x4096xf32>
    %7 = stablehlo.multiply %4, %6 : tensor<2048x4096xf32>
    return %0, %7 : tensor<2048x4096xi32>, tensor<2048x4096xf32>
  }
}
