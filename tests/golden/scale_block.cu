// Source of tests/golden/scale_block_sm100a.ptx (see make_ptx.sh): the smallest generated block.
extern "C" __global__ void dgen_scale_block(const float *x, float *y, float gain, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = x[i] * gain;
}
