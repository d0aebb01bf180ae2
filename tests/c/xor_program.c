/* A user program written against the public header the way the reference's documentation shows it (designated
 * arguments through the new_spingalett / layer / train / forward / save_spingalett macros): the exclusive-or problem
 * with a mean-squared-error loss, FOO52 hidden units, a sigmoid output and AdamW with weight decay -- the request mix
 * that needs every part of the train() surface beyond cross-entropy + Adam.  Prints one line per pattern and exits 0
 * only if all four are learnt and the saved file gives the same outputs after load_spingalett. */
#include <Spingalett/Spingalett.h>
#include <math.h>
#include <stdio.h>

static size_t calls = 0;
static bool progress(NeuralNetwork *net, size_t epoch, float error)
{
    (void)net;
    calls++;
    printf("callback epoch %zu error %.6f\n", epoch, (double)error);
    return error < 1e-5f;
}

int main(void)
{
    float in[] = { 0.f, 0.f, 0.f, 1.f, 1.f, 0.f, 1.f, 1.f };
    float want[] = { 0.f, 1.f, 1.f, 0.f };
    spingalett_set_verbose(false);
    NeuralNetwork *nn = new_spingalett(.loss_func = LOSS_MSE);
    layer(nn, 2);
    layer(nn, 8, ACT_FOO52, WEIGHT_INITIALIZATION_HE);
    layer(nn, 1, ACT_SIGMOID, WEIGHT_INITIALIZATION_XAVIER);
    train(.net = nn, .training_mode = MODE_ARRAY, .training_strategy = STRATEGY_FULL_BATCH, .optimizer_type = OPTIMIZER_ADAMW,
          .inputs = in, .targets = want, .sample_count = 4, .epochs = 4000, .learning_rate = 0.01f, .weight_decay = 1e-4f,
          .callback = progress, .callback_interval = 2000);
    if (spingalett_last_error_code() != SPINGALETT_OK) { printf("train failed: %s\n", spingalett_last_error_message()); return 2; }
    int ok = 0;
    float kept[4];
    for (int i = 0; i < 4; i++) {
        float *out = forward(.net = nn, .input = &in[2 * i]);
        if (!out) { printf("forward failed: %s\n", spingalett_last_error_message()); return 3; }
        kept[i] = out[0];
        const bool good = fabsf(out[0] - want[i]) < 0.1f;
        printf("%s in=[%.0f, %.0f] target=%.0f output=%.4f\n", good ? "OK" : "FAIL", (double)in[2 * i], (double)in[2 * i + 1],
               (double)want[i], (double)out[0]);
        ok += good;
    }
    save_spingalett(.net = nn, .filename = "xor_program_model", .precision = PRECISION_FLOAT32);
    free_network(nn);
    NeuralNetwork *back = load_spingalett("xor_program_model.nn");
    if (!back) { printf("load failed\n"); return 4; }
    int same = 0;
    for (int i = 0; i < 4; i++) {
        float *out = forward(.net = back, .input = &in[2 * i]);
        same += out && fabsf(out[0] - kept[i]) < 1e-6f;
    }
    free_network(back);
    printf("passed %d/4, reloaded %d/4, callbacks %zu\n", ok, same, calls);
    return ok == 4 && same == 4 && calls >= 1 ? 0 : 1;
}
