from ._edge_embed import edge_embed
from ._activation import Activation
from ._gate import Gate
from ._fc import FullyConnectedNet, bessel, normalize2mom_constant
from ._linear_gate import LinearGate
from ._interaction import InteractionBlock, neighbor_list_pbc, radius_graph_pbc

__all__ = ["Activation", "Gate", "LinearGate", "edge_embed", "FullyConnectedNet", "bessel", "normalize2mom_constant", "InteractionBlock", "radius_graph_pbc", "neighbor_list_pbc"]
