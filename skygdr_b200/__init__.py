"""SkyGDR-B200: a Blackwell-native GPU-fabric scheduling runtime.

Applications register communication flows with a priority or a bandwidth
goal; a C++ control daemon turns link and flow signals into per-flow byte
budgets every few milliseconds; hand-written sm_100a kernels move the bytes
and check those budgets chunk by chunk.

Sub-packages: ``control`` (daemon, protocol, policies, simulator),
``ops`` (kernels), ``models`` (Qwen3), ``parallel`` (peer memory, tensor
parallelism, prefill/decode disaggregation), ``utils``, ``cli``.
"""
__version__ = "0.1.0"
