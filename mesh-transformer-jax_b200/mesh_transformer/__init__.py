"""B200-native drop-in for the GPT-J forward / eval / decode path of
mesh_transformer (kingoflolz/mesh-transformer-jax): same module and class
names, compute in libmtj_b200's sm_100a kernels."""
