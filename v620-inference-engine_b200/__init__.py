"""qw-b200: a Blackwell-native inference engine for the 180B hybrid MoE
"Qwen3.8-Flash-Next" (GDN linear attention + QSA sparse attention + 4-stream
hyper-connections + 512 routed / 1 shared q4 experts + MTP head + host PLE table).

Layout of the package:

* ``models``   – shapes, shard math, q4 quantisation, n-gram hasher, PLE table,
                 weight synthesis / checkpoint loading, the fp32 torch oracle.
* ``ops``      – hand-written sm_100a CUDA kernels (``csrc/``) and their ctypes bindings.
* ``parallel`` – rank groups, NCCL baseline collectives, symmetric-memory fused collectives,
                 a CPU-rank backend for protocol and fault tests.
* ``engine``   – slots, buffers, decode graphs, prefill scheduler, speculative decoding, KV spill.
* ``session``  – prefix cache (block store + disk tier), samplers, the generate loop.
* ``server``   – the OpenAI-compatible ``qwserve`` HTTP server.
* ``native``   – C++ host runtime sources (core, CPU reference, session, C API shim).
* ``utils``    – logging, env/config flags, timers, NVML clocks sampling.
"""
__version__ = "0.1.0"
