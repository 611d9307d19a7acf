"""Forward stages of the chunked EMA (reference: kernels/ema_kernels/)."""
