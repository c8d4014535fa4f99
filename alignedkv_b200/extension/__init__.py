"""Host-side mirror of the reference's `extension` package (extension/KV_cache_cpp_extention.py,
extension/k_cache_file.py, extension/v_cache_file.py) on top of the sm_100a C-ABI library."""
