"""Drop-in for the reference's `torchac_cuda` extension module.

Same four functions, argument meaning and error behaviour as
LMCache/third_party/torchac_cuda/main.cpp:14-17 in the reference; the work is done by the
sm_100a kernels behind the C ABI (include/cachegen_b200.h).  Differences a caller can see:

  * launches go to torch's *current* stream of the tensors' device (the reference launches on the
    legacy default stream);
  * `encode_fast_new` reports a stream that outgrows its row of `output_buffer` (RuntimeError)
    instead of overrunning shared memory;
  * any number of channels works (the reference needs a power-of-two factor for its block size).

`import cachegen_b200.torchac_cuda as torchac_cuda`, or `cachegen_b200.compat.install()` to make
`import torchac_cuda` resolve here.
"""
import ctypes

import torch

from . import _lib

MAX_LP_ENCODE = 48   # torchac_kernel_enc_new.cu:6
MAX_LP_DECODE = 64   # torchac_kernel_dec_new.cu:6
MAX_BINS_SUPPORTED = 64  # cal_cdf.cu:7
MAX_TOKENS = _lib.CG_MAX_TOKENS_PER_STREAM


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


_status = {}


def _status_word(device):
    """One int32 status word per device, zeroed once and re-zeroed by whoever reads a non-zero value."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    w = _status.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = w
    return w


def calculate_cdf(input: torch.Tensor, max_bins: int) -> torch.Tensor:
    """int8 symbols [nlayers, ntokens, nchannels] -> int16 tables [nlayers, nchannels, max_bins + 1]
    (cal_cdf.cu:68-129)."""
    _check(input.is_cuda, "Input must be a CUDA tensor")
    _check(max_bins < MAX_BINS_SUPPORTED, f"Max bins must be less than {MAX_BINS_SUPPORTED}")
    _check(input.dim() == 3 and input.dtype in (torch.int8, torch.uint8), "expected an int8 tensor of rank 3")
    nlayers, ntokens, nchannels = input.shape
    out = torch.empty((nlayers, nchannels, max_bins + 1), dtype=torch.int16, device=input.device)
    with torch.cuda.device(input.device):
        rc = _lib.lib().cg_calculate_cdf(_ptr(input), _lib.strides3(input), nlayers, ntokens, nchannels,
                                         int(max_bins), _ptr(out), _stream(input))
    _lib.check(rc, "calculate_cdf")
    return out


def encode_fast_new(cdf: torch.Tensor, input_sym: torch.Tensor, output_buffer: torch.Tensor,
                    output_lengths: torch.Tensor) -> None:
    """Arithmetic-encodes every (layer, channel) stream of <= 256 tokens into its row of
    `output_buffer`, byte count into `output_lengths` (torchac_kernel_enc_new.cu:355-451)."""
    _check(cdf.is_cuda, "CDF should be on GPU")
    _check(input_sym.is_cuda, "Input symbols should be on GPU")
    _check(output_buffer.is_cuda, "Output buffer should be on GPU")
    _check(output_lengths.is_cuda, "Output lengths should be on GPU")
    _check(cdf.dim() == 3 and input_sym.dim() == 3 and output_buffer.dim() == 3 and output_lengths.dim() == 2,
           "expected cdf, input symbols and output buffer of rank 3 and output lengths of rank 2")
    _check(input_sym.dtype in (torch.int8, torch.uint8), "expected int8 input symbols")
    cs, ins, os_, ls = cdf.shape, input_sym.shape, output_buffer.shape, output_lengths.shape
    _check(cs[0] == ins[0], "CDF and input should have the same number of layers")
    _check(cs[1] == ins[2], "CDF and input should have the same number of layers")
    _check(os_[0] == cs[0], "Output buffer should have the same number of layers as CDF")
    _check(os_[1] == cs[1], "Output buffer should have the same number of channels as CDF")
    _check(ls[0] == cs[0], "Output lengths should have the same number of layers as CDF")
    _check(ls[1] == cs[1], "Output lengths should have the same number of channels as CDF")
    nlayers, nchannels, lp = cs
    ntokens = ins[1]
    _check(ntokens <= MAX_TOKENS, f"Number of tokens should be less than or equal to {MAX_TOKENS}")
    _check(lp <= MAX_LP_ENCODE, "CDF length should be less than MAX_LP")
    _check(cdf.is_contiguous() and output_buffer.is_contiguous() and output_lengths.is_contiguous(),
           "cdf, output buffer and output lengths must be contiguous")
    _check(output_buffer.dtype == torch.uint8 and output_lengths.dtype == torch.int32 and
           cdf.dtype == torch.int16, "expected int16 cdf, uint8 output buffer, int32 output lengths")
    status = _status_word(cdf.device)
    with torch.cuda.device(cdf.device):
        rc = _lib.lib().cg_encode_padded(_ptr(cdf), _ptr(input_sym), _lib.strides3(input_sym), nlayers, ntokens,
                                         nchannels, lp, _ptr(output_buffer), os_[2], _ptr(output_lengths),
                                         _ptr(status), _stream(cdf))
    _lib.check(rc, "encode_fast_new")


def check_status(device=None) -> None:
    """Synchronises and raises if a kernel of this module reported a problem since the last check
    (an encoded stream longer than its buffer row, malformed lengths, an out-of-table symbol)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _status_word(device)
    bits = int(w.item())
    if bits:
        w.zero_()
        raise RuntimeError("torchac_cuda: " + _lib.status_text(bits))


def decode_fast_new(cdf: torch.Tensor, bytestreams: torch.Tensor, lengths: torch.Tensor,
                    output: torch.Tensor) -> None:
    """Decodes padded streams [nlayers, nchannels, row] + int32 lengths into uint8 symbols
    [nlayers, ntokens, nchannels] (torchac_kernel_dec_new.cu:314-393)."""
    _check(cdf.is_cuda, "CDF should be on GPU")
    _check(bytestreams.is_cuda, "Bytestreams should be on GPU")
    _check(lengths.is_cuda, "Lengths should be on GPU")
    _check(output.is_cuda, "Output should be on GPU")
    _check(cdf.dim() == 3 and bytestreams.dim() == 3 and lengths.dim() == 2 and output.dim() == 3,
           "expected cdf, bytestreams and output of rank 3 and lengths of rank 2")
    _check(bytestreams.dtype == torch.uint8 and output.dtype == torch.uint8, "expected uint8 bytestreams and output")
    cs, bs, ls, os_ = cdf.shape, bytestreams.shape, lengths.shape, output.shape
    _check(cs[0] == bs[0], "CDF and bytestreams should have the same number of layers")
    _check(cs[1] == bs[1], "CDF and bytestreams should have the same number of channels")
    _check(cs[0] == ls[0], "CDF and lengths should have the same number of layers")
    _check(cs[1] == ls[1], "CDF and lengths should have the same number of channels")
    _check(cs[0] == os_[0], "CDF and output should have the same number of layers")
    _check(cs[1] == os_[2], "CDF and output should have the same number of channels")
    nlayers, nchannels, lp = cs
    ntokens = os_[1]
    _check(ntokens <= MAX_TOKENS, f"Number of tokens should be less than or equal to {MAX_TOKENS}")
    _check(lp <= MAX_LP_DECODE, f"CDF should have at most {MAX_LP_DECODE} Lps")
    _check(cdf.is_contiguous() and bytestreams.is_contiguous() and lengths.is_contiguous(),
           "cdf, bytestreams and lengths must be contiguous")
    _check(lengths.dtype == torch.int32 and cdf.dtype == torch.int16, "expected int16 cdf and int32 lengths")
    status = _status_word(cdf.device)
    with torch.cuda.device(cdf.device):
        rc = _lib.lib().cg_decode_padded(_ptr(cdf), _ptr(bytestreams), bs[2], _ptr(lengths), _ptr(output),
                                         _lib.strides3(output), nlayers, ntokens, nchannels, lp, _ptr(status),
                                         _stream(cdf))
    _lib.check(rc, "decode_fast_new")


def _decode_prefsum(entry: str, cdf, bytestreams, lengths_prefsum, output) -> None:
    _check(cdf.is_cuda, "CDF should be on GPU")
    _check(bytestreams.is_cuda, "Bytestreams should be on GPU")
    _check(lengths_prefsum.is_cuda, "Lengths should be on GPU")
    _check(output.is_cuda, "Output should be on GPU")
    _check(cdf.dim() == 3 and lengths_prefsum.dim() == 2 and output.dim() == 3,
           "expected cdf and output of rank 3 and prefix sums of rank 2")
    _check(bytestreams.dtype == torch.uint8 and output.dtype == torch.uint8, "expected uint8 bytestreams and output")
    cs, ls, os_ = cdf.shape, lengths_prefsum.shape, output.shape
    _check(cs[0] == ls[0], "CDF and lengths should have the same number of layers")
    _check(cs[1] == ls[1], "CDF and lengths should have the same number of channels")
    _check(cs[0] == os_[0], "CDF and output should have the same number of layers")
    _check(cs[1] == os_[2], "CDF and output should have the same number of channels")
    nlayers, nchannels, lp = cs
    ntokens = os_[1]
    _check(ntokens <= MAX_TOKENS, f"Number of tokens should be less than or equal to{MAX_TOKENS}")
    _check(lp <= MAX_LP_DECODE, f"CDF should have at most{MAX_LP_DECODE}Lps")
    _check(cdf.is_contiguous() and bytestreams.is_contiguous() and lengths_prefsum.is_contiguous(),
           "cdf, bytestreams and lengths must be contiguous")
    _check(lengths_prefsum.dtype == torch.int64 and cdf.dtype == torch.int16 and bytestreams.dim() == 1,
           "expected int16 cdf, 1-D bytestreams and int64 prefix sums")
    status = _status_word(cdf.device)
    with torch.cuda.device(cdf.device):
        rc = getattr(_lib.lib(), entry)(_ptr(cdf), _ptr(bytestreams), bytestreams.numel(), _ptr(lengths_prefsum),
                                        _ptr(output), _lib.strides3(output), nlayers, ntokens, nchannels, lp,
                                        _ptr(status), _stream(cdf))
    _lib.check(rc, "decode_fast_prefsum")


def decode_fast_prefsum(cdf: torch.Tensor, bytestreams: torch.Tensor, lengths_prefsum: torch.Tensor,
                        output: torch.Tensor) -> None:
    """Decodes back-to-back streams located by an inclusive int64 prefix sum of their lengths into
    uint8 symbols [nlayers, ntokens, nchannels], strided output allowed
    (torchac_kernel_dec_new.cu:403-479)."""
    _decode_prefsum("cg_decode_prefsum", cdf, bytestreams, lengths_prefsum, output)


def decode_fast_prefsum_warp(cdf: torch.Tensor, bytestreams: torch.Tensor, lengths_prefsum: torch.Tensor,
                             output: torch.Tensor) -> None:
    """decode_fast_prefsum on the one-warp-per-stream kernel (tables of at most 33 entries): the same
    symbols, several times slower; exists so that the two layouts can be compared on the same input."""
    _decode_prefsum("cg_decode_prefsum_warp", cdf, bytestreams, lengths_prefsum, output)
