module @jit_f {
  func.func public @main(%arg0: tensor<6x8xi32>, %arg1: tensor<6x2xi32>) -> tensor<6x6xi32> {
    %0 = stablehlo.slice %arg0 [0:6, 1:8:2] : (tensor<6x8xi32>) -> tensor<6x4xi32>
    %1 = stablehlo.concatenate %0, %arg1, dim = 1 : (tensor<6x4xi32>, tensor<6x2xi32>) -> tensor<6x6xi32>
    %c = stablehlo.constant dense<3> : tensor<i32>
    %2 = stablehlo.broadcast_in_dim %c, dims = [] : (tensor<i32>) -> tensor<6x6xi32>
    %3 = stablehlo.shift_right_logical %1, %2 : tensor<6x6xi32>
    return %3 : tensor<6x6xi32>
  }
}
