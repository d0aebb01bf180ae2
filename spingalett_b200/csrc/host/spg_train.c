/* train(): placeholder until the GPU training step lands in this file. */
#include "spg_internal.h"

void spg_train_release(spg_net *n) { (void)n; }

void train_struct_arguments(TrainArgs args)
{
    (void)args;
    spg_set_error(SPINGALETT_ERR_INVALID, "train: not available in this build yet");
}
