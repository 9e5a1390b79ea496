"""Architecture-specific callers of the coded path.  Only the MoE block of the
reference's qwen3_5_moe plugin lives here: the model skeleton, loaders and
attention of the reference's plugins are outside the coded-projection path."""
