// Image inputs of vision-language models, router side.
//
// Same job as the image branch of the reference's validation (router/src/validation.rs:570-863,
// config.rs:378-421): the `inputs` string may embed images in markdown form `![alt](url)`; the
// validator splits it into text and image chunks, fetches each image (data: URIs with base64
// payload, or plain http:// URLs), checks its size, reads its dimensions from the file header and
// accounts for the placeholder tokens the model will spend on it.
#pragma once
#include <cstdint>
#include <optional>
#include <string>
#include <vector>

#include "json.hpp"
#include "pb.hpp"

namespace images {

struct Piece {
  bool is_image = false;
  std::string text;   // text piece, or the URL of an image piece
};

// "a ![](u1) b" -> [text "a ", image u1, text " b"]; text without images gives one text piece.
std::vector<Piece> split_markdown(const std::string& inputs);

struct Fetched {
  std::string data;
  std::string mimetype;
  uint32_t width = 0, height = 0;
};

// Throws std::runtime_error with a user-facing message (bad URI, unsupported scheme, too large,
// unknown format).  `max_bytes` bounds the decoded size.
Fetched fetch(const std::string& url, size_t max_bytes);

std::string base64_decode(const std::string& s);

// (width, height) from a PNG / JPEG / GIF / WebP / BMP header; nullopt when the format is unknown.
std::optional<std::pair<uint32_t, uint32_t>> dimensions(const std::string& bytes, std::string* mimetype);

// Placeholder tokens one image costs for the model described by `config` (config.json of the
// checkpoint); 0 when the model takes no images.
uint32_t tokens_per_image(const json::Value& config, uint32_t width, uint32_t height);

// Stable pseudo token id for position `i` of an image: the prefix cache keys on token ids, and two
// different images must not share a prefix.  Ids live above any vocabulary (top bit set).
uint32_t placeholder_id(const std::string& data, uint32_t i);

}  // namespace images
