from tensor_parallel_b200.utils.nested import nested_compare, nested_flatten, nested_map, nested_pack
from tensor_parallel_b200.utils.tied import check_lora, find_tied_weight_aliases

__all__ = [
    "nested_compare",
    "nested_flatten",
    "nested_map",
    "nested_pack",
    "check_lora",
    "find_tied_weight_aliases",
]
