"""The built-in parts, registered by kind."""

from tandem_b200.parts.attention import PagedAttention
from tandem_b200.parts.block import ConnectedBlock, ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock
from tandem_b200.parts.connection import DepthAverage, StreamLink
from tandem_b200.parts.convolution import ShortConvolution
from tandem_b200.parts.latent_attention import LatentAttention
from tandem_b200.parts.mlp import DenseMLP, GatedMLP, RoutedMLP
from tandem_b200.parts.norm import GroupRMSNorm, RMSNorm
from tandem_b200.parts.recurrence import DecayRecurrence, SelectiveRecurrence
from tandem_b200.parts.rope import NoPosition, RotaryTable
from tandem_b200.parts.sink_attention import SinkAttention
from tandem_b200.parts.window_attention import WindowAttention
from tandem_b200.registry import register_part

register_part("mixer", "attention", PagedAttention)
register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("norm", "rmsnorm", RMSNorm)
register_part("position", "rope", RotaryTable)
register_part("position", "none", NoPosition)
register_part("block", "prenorm", PreNormBlock)
register_part("mixer", "sink_attention", SinkAttention)
register_part("mixer", "decay_recurrence", DecayRecurrence)
register_part("feed_forward", "dense_mlp", DenseMLP)
register_part("block", "parallel", ParallelBlock)
register_part("mixer", "selective_recurrence", SelectiveRecurrence)
register_part("mixer", "latent_attention", LatentAttention)
register_part("feed_forward", "routed_mlp", RoutedMLP)
register_part("connection", "stream_link", StreamLink)
register_part("block", "connected", ConnectedBlock)
register_part("norm", "group_rmsnorm", GroupRMSNorm)
register_part("mixer", "short_convolution", ShortConvolution)
register_part("connection", "depth_average", DepthAverage)
register_part("block", "postnorm", PostNormBlock)
register_part("mixer", "window_attention", WindowAttention)
register_part("block", "sandwich", SandwichBlock)
