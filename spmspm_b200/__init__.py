"""B200 (sm_100a) implementation of the SpInfer bitmap-v3 sparse SpMM path, behind the reference's interface."""
from .api import (init, release, BitmapMatrix, HostEncoded, SpmmError, device_status, encode_device, init_sparse_matrix_a_bitmap,
                  our_gen_sparse_matrix_bin_file, reset_device_status, set_schedule, SCHEDULE_AUTO, SCHEDULE_BALANCED, SCHEDULE_STATIC, splitk_reduce, spmm, spmm_allgather, spmm_allreduce, allreduce_finish, wait_flags, linear, ACT_NONE, ACT_RELU, launch_count, init_sparse_matrix_a_bitmap_v6_b, decode_operand_b, spmspm, spmm_noalloc, spmm_splitk_api_bitmap_v3,
                  suggest_split_k, to_device, bin_file_names, load_bin_files, read_rank_lists, write_rank_lists)

__all__ = ["init", "release", "BitmapMatrix", "HostEncoded", "SpmmError", "device_status", "encode_device",
           "init_sparse_matrix_a_bitmap", "our_gen_sparse_matrix_bin_file", "reset_device_status", "set_schedule", "SCHEDULE_AUTO", "SCHEDULE_BALANCED", "SCHEDULE_STATIC", "splitk_reduce",
           "spmm", "spmm_allgather", "spmm_allreduce", "allreduce_finish", "linear", "ACT_NONE", "ACT_RELU", "launch_count", "init_sparse_matrix_a_bitmap_v6_b", "decode_operand_b", "spmspm", "spmm_noalloc", "wait_flags", "spmm_splitk_api_bitmap_v3", "suggest_split_k", "to_device",
           "bin_file_names", "load_bin_files", "read_rank_lists", "write_rank_lists"]
