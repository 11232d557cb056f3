"""Small seeded cases shared by the fixture generator, the CPU tests and the GPU parity tests."""
from flashmoe_b200.jit import ActivationType as A, DataType as D, MLPType as M
from flashmoe_b200.workloads import Workload

# name -> Workload.  Sizes are chosen so that the CPU oracle finishes each in well under a second.
GOLDEN_CASES = {
    # gated SiLU, k = 2, nothing dropped
    "bf16_gated_k2": Workload("bf16_gated_k2", 96, 256, 384, 8, 2, D.BF16, M.GATED, A.SILU, seed=11),
    # k = 1, ragged tile (S not a multiple of anything), biases on
    "bf16_gated_k1_bias": Workload("bf16_gated_k1_bias", 77, 128, 256, 16, 1, D.BF16, M.GATED, A.SILU,
                                   seed=12, bias_std=0.5),
    # reference-default capacity: tokens beyond ceil(S/E)*k are dropped
    "bf16_drop": Workload("bf16_drop", 128, 128, 128, 8, 2, D.BF16, M.GATED, A.SILU, seed=13,
                          capacity=20, zipf_bias=True),
    # plain MLP, GELU, many experts, k = 8 (fine-grained shape)
    "bf16_vanilla_gelu_k8": Workload("bf16_vanilla_gelu_k8", 64, 256, 256, 64, 8, D.BF16, M.VANILLA,
                                     A.GELU, seed=14, bias_std=0.1),
    # fp16, ReLU
    "fp16_gated_relu": Workload("fp16_gated_relu", 50, 192, 320, 8, 2, D.FP16, M.GATED, A.RELU, seed=15),
    # fp32 layers (three BF16 planes per operand on the tensor cores), tolerance 1e-5
    "fp32_gated_k2": Workload("fp32_gated_k2", 96, 256, 384, 8, 2, D.FP32, M.GATED, A.SILU, seed=17,
                              bias_std=0.2),
    "fp32_vanilla_gelu_k4": Workload("fp32_vanilla_gelu_k4", 80, 192, 256, 16, 4, D.FP32, M.VANILLA, A.GELU,
                                     seed=18),
    # an expert with more than one M tile of rows
    "bf16_two_mtiles": Workload("bf16_two_mtiles", 400, 128, 128, 8, 2, D.BF16, M.GATED, A.SILU, seed=16,
                                zipf_bias=True),
}
# router-only cases (any dtype the router takes; H is a multiple of 64 because the routing table
# lives in an MoE context; 960 and 192 leave the router's last 32-lane pass ragged)
ROUTER_CASES = {
    "r_fp32_e8_k2": Workload("r_fp32_e8_k2", 128, 1024, 64, 8, 2, D.FP32, seed=21),
    "r_bf16_e16_k1": Workload("r_bf16_e16_k1", 200, 512, 64, 16, 1, D.BF16, seed=22),
    "r_bf16_e128_k8": Workload("r_bf16_e128_k8", 130, 2048, 64, 128, 8, D.BF16, seed=23),
    "r_bf16_e256_k8_zipf": Workload("r_bf16_e256_k8_zipf", 96, 960, 64, 256, 8, D.BF16, seed=24,
                                    zipf_bias=True, capacity=6),
    "r_fp16_e24_k3": Workload("r_fp16_e24_k3", 33, 192, 64, 24, 3, D.FP16, seed=25),
    "r_bf16_ties": Workload("r_bf16_ties", 64, 64, 64, 16, 4, D.BF16, seed=26),
}
