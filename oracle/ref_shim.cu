/*
 * TEST INFRASTRUCTURE — C entry points around the reference's own GPU kernels.
 *
 * oracle/Makefile compiles this file together with the reference's source/clusterKernels.cu and
 * source/basicOps.cu, where they lie in the mounted reference tree, into oracle/_ref/libcnref.so.
 * Nothing of the reference is copied: this shim only wraps raw device pointers in the reference's
 * `Matrix` descriptor (source/basicOps.cuh:25-42) and calls the reference's host launchers, so that
 * tests and the golden-vector generator can run the unmodified kernels on the same buffers as the
 * new kernels.  The product library never links or loads it.
 */
#include <basicOps.cuh>
#include <clusterKernels.cuh>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

static Matrix wrap(float *data, int rows, int cols)
{
    Matrix m;
    memset(&m, 0, sizeof(m));
    m.rows = rows;
    m.cols = cols;
    m.size = rows * cols;
    m.bytes = (size_t)rows * cols * sizeof(float);
    m.data = data;
    return m;
}

extern "C" {

/* source/basicOps.cu:1163-1168 -> kCompression_8bit */
int ref_compression_8bit(float *d_tbl, float *d_A, float precision, int n, unsigned char *d_out)
{
    Matrix tbl = wrap(d_tbl, 126, 1);
    Matrix A = wrap(d_A, n, 1);
    Matrix out = wrap(0, n, 1);
    out.char_data = d_out;
    compression_8bit(&tbl, &A, precision, &out);
    return (int)cudaDeviceSynchronize();
}

/* source/basicOps.cu:1172-1176 -> kDecompression_8bit */
int ref_decompression_8bit(float *d_tbl, unsigned char *d_codes, float precision, int n, float *d_out)
{
    Matrix tbl = wrap(d_tbl, 126, 1);
    Matrix A = wrap(0, n, 1);
    A.char_data = d_codes;
    Matrix out = wrap(d_out, n, 1);
    decompression_8bit(&tbl, &A, precision, &out);
    return (int)cudaDeviceSynchronize();
}

/* The same two launchers without the device synchronisation, for timing a series of launches with events */
void ref_compression_8bit_async(float *d_tbl, float *d_A, float precision, int n, unsigned char *d_out)
{
    Matrix tbl = wrap(d_tbl, 126, 1);
    Matrix A = wrap(d_A, n, 1);
    Matrix out = wrap(0, n, 1);
    out.char_data = d_out;
    compression_8bit(&tbl, &A, precision, &out);
}

void ref_decompression_8bit_async(float *d_tbl, unsigned char *d_codes, float precision, int n, float *d_out)
{
    Matrix tbl = wrap(d_tbl, 126, 1);
    Matrix A = wrap(0, n, 1);
    A.char_data = d_codes;
    Matrix out = wrap(d_out, n, 1);
    decompression_8bit(&tbl, &A, precision, &out);
}

/* abs + max: source/basicOps.cu:810-822,1076-1081 */
float ref_absmax(float *d_A, float *d_tmp, int n)
{
    Matrix A = wrap(d_A, n, 1);
    Matrix t = wrap(d_tmp, n, 1);
    abs(&A, &t);
    return max(&t);
}

/* source/basicOps.cu:966-974 */
int ref_addMatrixVector(float *d_A, float *d_v, float *d_out, int rows, int cols)
{
    Matrix A = wrap(d_A, rows, cols), v = wrap(d_v, 1, cols), out = wrap(d_out, rows, cols);
    addMatrixVector(&A, &v, &out);
    return (int)cudaDeviceSynchronize();
}

/* source/basicOps.cu:1212-1216, 672-676 */
int ref_rectified_linear(float *d_A, float *d_out, int n)
{
    Matrix A = wrap(d_A, n, 1), out = wrap(d_out, n, 1);
    rectified_linear(&A, &out);
    return (int)cudaDeviceSynchronize();
}

int ref_logistic(float *d_A, float *d_out, int n)
{
    Matrix A = wrap(d_A, n, 1), out = wrap(d_out, n, 1);
    logistic(&A, &out);
    return (int)cudaDeviceSynchronize();
}

/* source/basicOps.cu:1287-1299 */
int ref_maxout(float *d_A, float *d_out, float *d_arg, int rows, int cols, int level)
{
    Matrix A = wrap(d_A, rows, cols), out = wrap(d_out, rows, cols / level), arg = wrap(d_arg, rows, cols / level);
    maxout(&A, &out, &arg, level);
    return (int)cudaDeviceSynchronize();
}

/* source/basicOps.cu:108-127: row-major <-> col-major on the device */
int ref_to_col_major(float *d_A, float *d_out, int rows, int cols)
{
    Matrix A = wrap(d_A, rows, cols), out = wrap(d_out, rows, cols);
    to_col_major(&A, &out);
    return (int)cudaDeviceSynchronize();
}

/* source/basicOps.cu:193-197 (limits +-4*sqrt(6/(in+out)) applied to uniforms already in the buffer) */
int ref_uniformSqrtWeight(float *d_A, int rows, int cols, int in, int out_total)
{
    Matrix A = wrap(d_A, rows, cols);
    uniformSqrtWeight(&A, in, out_total);
    return (int)cudaDeviceSynchronize();
}

}  /* extern "C" */
