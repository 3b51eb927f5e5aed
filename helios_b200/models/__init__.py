"""Plan builders; importing this package registers the architectures."""
from . import dense_decoder, fobanex, gebasun, mizerax, zokelix
from .dense_decoder import build_dense_decoder_plan
from .fobanex import build_fobanex_plan
from .gebasun import build_gebasun_plan
from .mizerax import build_mizerax_plan
from .zokelix import build_zokelix_plan

__all__ = ["build_dense_decoder_plan", "build_fobanex_plan", "fobanex", "build_gebasun_plan", "gebasun", "build_mizerax_plan", "build_zokelix_plan", "dense_decoder", "mizerax",
           "zokelix"]
