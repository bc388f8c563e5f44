"""DP gradient engines.

``clipping``  – the functional reference engine: ``vmap(grad)`` per-example
                gradients, batched clip, weighted sum (runs on CPU and GPU).
``fused``     – the explicit-batch B200 engine: one forward/backward per
                microbatch with captured layer activations and output
                gradients, per-example norms from fused kernels, and a
                clip-weighted weight-gradient GEMM whose epilogue
                reduce-scatters into the owning rank's shard.
"""
