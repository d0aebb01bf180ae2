/*
 * Feature macros of this build (the reference generates this file from
 * Include/Spingalett/Spingalett.Config.h.in).  This library computes on CUDA
 * only: there is no OpenMP, OpenBLAS or other CPU compute path behind it.
 */
#pragma once
#define SPINGALETT_HAS_CUDA
#define SPINGALETT_B200 1
