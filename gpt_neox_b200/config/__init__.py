from .args import NeoXArgs, expand_attention_types, resource_pool, read_hostfile
from .schema import FIELDS, GROUPS, ATTENTION_TYPE_CHOICES

__all__ = ["NeoXArgs", "FIELDS", "GROUPS", "ATTENTION_TYPE_CHOICES", "expand_attention_types", "resource_pool",
           "read_hostfile"]
