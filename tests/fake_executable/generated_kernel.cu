// TEST INFRASTRUCTURE.  Stands in for a kernel the DISC compiler generated (a kLoop
// fusion): y = a * x + b.  The tests build device images from it with nvcc and
// launch it through ral_kernel_launch, as a compiled executable would.
extern "C" __global__ void axpb(const float* x, float* y, float a, float b, long n) {
  long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (i < n) y[i] = a * x[i] + b;
}
