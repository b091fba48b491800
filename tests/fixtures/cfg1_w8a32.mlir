module @jit_f attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<32x1024xf32>, %arg1: tensor<1024x1024xi8>, %arg2: tensor<1024xf32>) -> (tensor<32x1024xf32> {jax.result_info = "result"}) {
    %0 = stablehlo.convert %arg1 : (tensor<1024x1024xi8>) -> tensor<1024x1024xf32>
    %1 = stablehlo.broadcast_in_dim %arg2, dims = [1] : (tensor<1024xf32>) -> tensor<1x1024xf32>
    %2 = stablehlo.broadcast_in_dim %1, dims = [0, 1] : (tensor<1x1024xf32>) -> tensor<1024x1024xf32>
    %3 = stablehlo.multiply %0, %2 : tensor<1024x1024xf32>
    %4 = stablehlo.dot_general %arg0, %3, contracting_dims = [1] x [0], precision = [DEFAULT, DEFAULT] : (tensor<32x1024xf32>, tensor<1024x1024xf32>) -> tensor<32x1024xf32>
    return %4 : tensor<32x1024xf32>
  }
}
