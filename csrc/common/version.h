// Library and wire-protocol versions (reference csrc/common/Version.hpp:3-15).
#pragma once

#define MCCL_VERSION_MAJOR 0
#define MCCL_VERSION_MINOR 5
#define MCCL_VERSION_PATCH 0
#define MCCL_VERSION_STRING "0.5.0"
// Version carried in every host-transport frame header and in the handshake.
#define MCCL_PROTOCOL_VERSION 5
