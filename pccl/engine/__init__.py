"""``pccl.engine``: Engine(rank, world) with initEngine / regOp / exeOp / exportEndpoint / joinCluster /
exitCluster, and ``engine_c`` (the raw native module, the reference's ``pccl.engine_c``)."""
from pccl_b200.engine import *  # noqa: F401,F403
from pccl_b200.engine import engine_c  # noqa: F401
