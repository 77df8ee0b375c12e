"""B200 (sm_100a) implementation of the nvfp4_training interface."""
