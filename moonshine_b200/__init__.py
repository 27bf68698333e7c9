"""B200-native routed-MoE path of the Moonshine Kimi-K3 engine.

``ops``   - the reference's C operator interface (``k3_rocm_*``) on torch tensors
``layer`` - slot table + fused layer (router, dispatch, grouped experts, combine)
``ep``    - expert-parallel layer over torch.distributed
``synth`` - seeded synthetic tensors
"""
__version__ = "0.1.0"
