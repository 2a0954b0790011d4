"""Peer plane of the engine service: links between daemons, rendezvous object sends, groups, collectives."""
from .core import CollectiveQueue, PeerCore
from .groups import GroupRecord, GroupTable
from .transports import FaultPlan, MemLink
