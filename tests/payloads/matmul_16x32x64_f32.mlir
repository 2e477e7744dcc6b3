// f32 linalg.matmul on tensor arguments, accumulating into the third argument in place.
module {
  func.func @main(%arg0: tensor<16x64xf32>, %arg1: tensor<64x32xf32>, %out: tensor<16x32xf32>) {
    %0 = arith.constant 0.000000e+00 : f32
    %1 = linalg.fill ins(%0 : f32) outs(%out : tensor<16x32xf32>) -> tensor<16x32xf32>
    %2 = linalg.matmul ins(%arg0, %arg1 : tensor<16x64xf32>, tensor<64x32xf32>) outs(%out : tensor<16x32xf32>) -> tensor<16x32xf32>
    return
  }
}
