// Shared between the recurrent-mixer kernels and the host: how many columns of a head's state matrix
// one thread block owns.  The matrix memory keeps its normaliser and stabiliser once per such block,
// so the size of a request's state depends on it.
#pragma once
#define SANDY_MATRIX_STATE_COLS 16
