// The reference's sources ask for the CUDA runtime header; under the host emulation (ref_emu.h) every
// CUDA name they use is already defined, so this header is empty on purpose.
#pragma once
