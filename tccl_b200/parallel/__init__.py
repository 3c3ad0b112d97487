from .tree import build_double_tree, build_tree, get_parents_and_children, tree_depths, tree_neighbours
from .simulate import simulate_double_tree_all_reduce
