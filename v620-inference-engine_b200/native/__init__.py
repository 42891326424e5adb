"""Native C++ host runtime (libqw_host.so): n-gram ids, PLE table, safetensors, block store + disk
tier, host sampler, chunker, thread pool; and the C API shim (libqw_engine.so)."""
