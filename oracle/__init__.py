"""CPU oracle for the quantized MoE FFN path (test infrastructure, see moe_oracle.cpp)."""
