# Applied by oracle/Makefile to a scratch copy (oracle/_ref/mhsa_fp32_patched.c) of the
# first 1747 lines of the reference's lib/sources/pulp_mhsa_fp32.c, which does not
# compile as shipped (half-finished refactor).  Each expression repairs one class of
# compile error without changing the arithmetic; the last-but-one sets the `t` flag the
# reference leaves uninitialised (lib/sources/pulp_mhsa_fp32.c:152-158).
s/int t_axes = \{1, 0\};/int t_axes[] = {1, 0};/
s/^(\s*)dims(\[\])? = \{([^,]+), ([^}]+)\};/\1dims[0] = \3; dims[1] = \4;/
s/int dims\[\] = \{E \* L\};/int dims1[] = {E * L};/
s/struct vect_sum_args vect_sum_args;/struct array_broadcast_sum_fp32_args vect_sum_args;/
s/op_1_dims = dims;/op_1_dims = dims1;/
s/op_2_dims = dims;/op_2_dims = dims1;/
s/\.matrix = /.in_matrix = /
s/\.transp_matrix = /.out_matrix = /
s/(mm_bias_add_args_[qkv])\.W = L;/\1.W = L; \1.t = 1;/
