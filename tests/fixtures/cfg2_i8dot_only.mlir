module @jit_f {
  func.func public @main(%arg0: tensor<256x512xui8>, %arg1: tensor<512x128xi8>) -> tensor<256x128xi32> {
    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0] : (tensor<256x512xui8>, tensor<512x128xi8>) -> tensor<256x128xi32>
    return %0 : tensor<256x128xi32>
  }
}
