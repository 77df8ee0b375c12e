"""Host-side orchestration of the NVFP4 training path; every kernel lives in libnvfp4_b200.so."""
