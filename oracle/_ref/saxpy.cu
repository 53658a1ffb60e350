__global__ void saxpy(float *y, float *x, float a, int n)
{
    int idx = threadIdx.x + blockIdx.x * blockDim.x;
    if (idx < n)
        y[idx] = a * x[idx] + y[idx];
}
