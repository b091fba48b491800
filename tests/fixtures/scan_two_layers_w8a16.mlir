module @jit_scan attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {
  func.func public @main(%arg0: tensor<256x512xbf16>, %arg1: tensor<2x512x512xi8>, %arg2: tensor<2x512xf32>) -> tensor<256x512xbf16> {
    %c = stablehlo.constant dense<0> : tensor<i32>
    %0:2 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg0) : tensor<i32>, tensor<256x512xbf16>
     cond {
      %c_1 = stablehlo.constant dense<2> : tensor<i32>
      %1 = stablehlo.compare  LT, %iterArg, %c_1,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    } do {
      %c_1 = stablehlo.constant dense<0> : tensor<i32>
      %1 = stablehlo.compare  LT, %iterArg, %c_1,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      %c_2 = stablehlo.constant dense<2> : tensor<i32>
      %2 = stablehlo.add %iterArg, %c_2 : tensor<i32>
      %3 = stablehlo.select %1, %2, %iterArg : tensor<i1>, tensor<i32>
      %4 = stablehlo.dynamic_slice %arg1, %3, %c_1, %c_1, sizes = [1, 512, 512] : (tensor<2x512x512xi8>, tensor<i32>, tensor<i32>, tensor<i32>) -> tensor<1x512x512xi8>
      %5 = stablehlo.reshape %4 : (tensor<1x512x512xi8>) -> tensor<512x512xi8>
      %6 = stablehlo.dynamic_slice %arg2, %3, %c_1, sizes = [1, 512] : (tensor<2x512xf32>, tensor<i32>, tensor<i32>) -> tensor<1x512xf32>
      %7 = stablehlo.reshape %6 : (tensor<1x512xf32>) -> tensor<512xf32>
      %8 = stablehlo.convert %5 : (tensor<512x512xi8>) -> tensor<512x512xbf16>
      %9 = stablehlo.convert %7 : (tensor<512xf32>) -> tensor<512xbf16>
      %10 = stablehlo.broadcast_in_dim %9, dims = [1] : (tensor<512xbf16>) -> tensor<512x512xbf16>
      %11 = stablehlo.multiply %8, %10 : tensor<512x512xbf16>
      %12 = stablehlo.dot_general %iterArg_0, %11, contracting_dims = [1] x [0] : (tensor<256x512xbf16>, tensor<512x512xbf16>) -> tensor<256x512xbf16>
      %c_3 = stablehlo.constant dense<1> : tensor<i32>
      %13 = stablehlo.add %iterArg, %c_3 : tensor<i32>
      stablehlo.return %13, %12 : tensor<i32>, tensor<256x512xbf16>
    }
    return %0#1 : tensor<256x512xbf16>
  }
}
