from .tree import (Static, Frozen, Vector, tensor_struct, model, tree_map, map_, map_m, zip_with, fold,  # noqa: F401
                            leaves, leaves_with_paths, with_leaves, count, grads, zero_grads, detach, requires_grad,
                            make_leaf_params, grad, functional_grad, scale, add, sub, all_, any_)
from .cast import cast_to, cast_like  # noqa: F401
from .schema import LeafSchema, schema_of, flatten, rebuild, diff_schemas  # noqa: F401
from .indexed import Select, IndexedList  # noqa: F401
