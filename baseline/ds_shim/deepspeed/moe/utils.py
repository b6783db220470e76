def is_moe_param(p):
    return getattr(p, "allreduce", True) is False


def split_params_into_different_moe_groups_for_optimizer(groups, *a, **k):
    return groups
