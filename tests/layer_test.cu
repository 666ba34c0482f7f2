// Trains the reference's 784-1200-1200-10 style MLP (here argv-sized) with the facade's Layer class on synthetic,
// linearly separable data and checks that the training error falls; also runs one step with dropout 0 and dumps the
// gradients so that tests/test_train_gpu.py can compare them with the CPU restatement.
#include <stdio.h>

#include <vector>

#include "../clusternet_b200/cpp/clusternet.hpp"

static void dump(const char *path, ClusterNet &gpu, Matrix *m)
{
    Matrix *h = gpu.to_host(m);
    FILE *f = fopen(path, "wb");
    fwrite(h->data, 4, h->size, f);
    fclose(f);
    free(h->data);
    free(h);
}

int main(int argc, char **argv)
{
    if (argc < 8) { printf("usage: layer_test codebook in hidden classes batch steps outdir\n"); return 1; }
    try {
        const int64_t in = atoll(argv[2]), hid = atoll(argv[3]), classes = atoll(argv[4]), B = atoll(argv[5]);
        const int steps = atoi(argv[6]);
        const std::string dir = argv[7];
        ClusterNet gpu(4321, argv[1]);
        // synthetic data: class = argmax of the first `classes` features
        Matrix *X = gpu.randn(B, in), *Xh = gpu.to_host(X), *yh = empty_cpu(B, 1);
        for (int64_t r = 0; r < B; ++r) {
            int best = 0;
            for (int64_t c = 1; c < classes; ++c) if (Xh->data[r * in + c] > Xh->data[r * in + best]) best = (int)c;
            yh->data[r] = (float)best;
        }
        Matrix *y = gpu.to_gpu(yh);
        Layer l0(in, B, Input, &gpu), l1(hid, Rectified_Linear), l2(hid, Rectified_Linear), l3(classes, Softmax);
        l0.PARALLELISM = DataParallelism;
        l0.DROPOUT = l1.DROPOUT = l2.DROPOUT = 0.0f;
        l0.link_with_next_layer(&l1); l1.link_with_next_layer(&l2); l2.link_with_next_layer(&l3);
        l3.target = y;
        cudaMemcpy(l0.activation->data, X->data, X->bytes, cudaMemcpyDeviceToDevice);
        dump((dir + "/X.bin").c_str(), gpu, X);
        dump((dir + "/y.bin").c_str(), gpu, y);
        dump((dir + "/w0.bin").c_str(), gpu, l0.w_next);
        dump((dir + "/w1.bin").c_str(), gpu, l1.w_next);
        dump((dir + "/w2.bin").c_str(), gpu, l2.w_next);
        // one step: forward, errors, gradients (dumped before any update)
        l0.forward(true);
        l0.backward_errors();
        dump((dir + "/probs.bin").c_str(), gpu, l3.out);
        dump((dir + "/g0.bin").c_str(), gpu, l0.w_grad_next);
        dump((dir + "/g1.bin").c_str(), gpu, l1.w_grad_next);
        dump((dir + "/g2.bin").c_str(), gpu, l2.w_grad_next);
        // training loop: the update of step t runs at the start of forward t+1, as in the reference
        float first = -1.f, last = -1.f;
        for (int s = 0; s < steps; ++s) {
            l0.forward(true);
            Matrix *p = gpu.to_host(l3.out);
            int wrong = 0;
            for (int64_t r = 0; r < B; ++r) {
                int best = 0;
                for (int64_t c = 1; c < classes; ++c) if (p->data[r * classes + c] > p->data[r * classes + best]) best = (int)c;
                wrong += best != (int)yh->data[r];
            }
            free(p->data); free(p);
            if (s == 0) first = wrong / (float)B;
            last = wrong / (float)B;
            l0.backward_errors();
        }
        printf("train error first %.4f last %.4f\n", first, last);
        if (!(last < 0.5f * first)) { printf("FAILED: training error did not fall\n"); return 1; }
        printf("All tests passed\n");
        return 0;
    } catch (const char *msg) {
        printf("exception: %s\n", msg);
        return 2;
    }
}
