#include "images.hpp"

#include <algorithm>
#include <cmath>

#include <arpa/inet.h>
#include <netdb.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

namespace images {

std::vector<Piece> split_markdown(const std::string& s) {
  std::vector<Piece> out;
  size_t pos = 0, text_start = 0;
  while (true) {
    const size_t bang = s.find("![", pos);
    if (bang == std::string::npos) break;
    const size_t close = s.find("](", bang + 2);
    if (close == std::string::npos) break;
    const size_t end = s.find(')', close + 2);
    if (end == std::string::npos) break;
    // the alt text must not contain a line break or another bracket pair start
    if (s.find('\n', bang) < close) {
      pos = bang + 2;
      continue;
    }
    if (bang > text_start) out.push_back({false, s.substr(text_start, bang - text_start)});
    out.push_back({true, s.substr(close + 2, end - close - 2)});
    pos = text_start = end + 1;
  }
  if (text_start < s.size() || out.empty()) out.push_back({false, s.substr(text_start)});
  return out;
}

std::string base64_decode(const std::string& s) {
  static int8_t table[256];
  static bool init = false;
  if (!init) {
    memset(table, -1, sizeof(table));
    const char* abc = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
    for (int i = 0; i < 64; ++i) table[static_cast<unsigned char>(abc[i])] = static_cast<int8_t>(i);
    table[static_cast<unsigned char>('-')] = 62;   // url-safe alphabet
    table[static_cast<unsigned char>('_')] = 63;
    init = true;
  }
  std::string out;
  out.reserve(s.size() * 3 / 4);
  uint32_t acc = 0;
  int bits = 0;
  for (unsigned char c : s) {
    if (c == '=' || c == '\n' || c == '\r' || c == ' ') continue;
    const int8_t v = table[c];
    if (v < 0) throw std::runtime_error("invalid base64 in image data URI");
    acc = (acc << 6) | static_cast<uint32_t>(v);
    bits += 6;
    if (bits >= 8) {
      bits -= 8;
      out.push_back(static_cast<char>((acc >> bits) & 0xff));
    }
  }
  return out;
}

namespace {

uint32_t be32(const unsigned char* p) { return (uint32_t(p[0]) << 24) | (uint32_t(p[1]) << 16) | (uint32_t(p[2]) << 8) | p[3]; }
uint32_t be16(const unsigned char* p) { return (uint32_t(p[0]) << 8) | p[1]; }
uint32_t le16(const unsigned char* p) { return uint32_t(p[0]) | (uint32_t(p[1]) << 8); }
uint32_t le32(const unsigned char* p) { return uint32_t(p[0]) | (uint32_t(p[1]) << 8) | (uint32_t(p[2]) << 16) | (uint32_t(p[3]) << 24); }

// Minimal HTTP/1.1 GET for plain http:// URLs (no TLS in this binary).
std::string http_get(const std::string& url, size_t max_bytes, std::string* content_type) {
  const std::string rest = url.substr(7);
  const size_t slash = rest.find('/');
  std::string hostport = slash == std::string::npos ? rest : rest.substr(0, slash);
  const std::string path = slash == std::string::npos ? "/" : rest.substr(slash);
  std::string host = hostport, port = "80";
  const size_t colon = hostport.rfind(':');
  if (colon != std::string::npos) {
    host = hostport.substr(0, colon);
    port = hostport.substr(colon + 1);
  }
  addrinfo hints{}, *res = nullptr;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host.c_str(), port.c_str(), &hints, &res) != 0 || res == nullptr)
    throw std::runtime_error("cannot resolve image host " + host);
  int fd = -1;
  for (addrinfo* a = res; a != nullptr; a = a->ai_next) {
    fd = socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (fd < 0) continue;
    timeval tv{10, 0};
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
    if (connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
    close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) throw std::runtime_error("cannot connect to image host " + host);
  const std::string req = "GET " + path + " HTTP/1.1\r\nHost: " + hostport + "\r\nConnection: close\r\nAccept: image/*\r\n\r\n";
  if (send(fd, req.data(), req.size(), 0) != static_cast<ssize_t>(req.size())) {
    close(fd);
    throw std::runtime_error("image request failed");
  }
  std::string raw;
  char buf[16384];
  while (true) {
    const ssize_t n = recv(fd, buf, sizeof(buf), 0);
    if (n <= 0) break;
    raw.append(buf, static_cast<size_t>(n));
    if (raw.size() > max_bytes + 65536) {
      close(fd);
      throw std::runtime_error("image is larger than the payload limit");
    }
  }
  close(fd);
  const size_t hdr_end = raw.find("\r\n\r\n");
  if (hdr_end == std::string::npos || raw.compare(0, 5, "HTTP/") != 0) throw std::runtime_error("malformed image response");
  const int status = atoi(raw.c_str() + 9);
  if (status != 200) throw std::runtime_error("image fetch returned HTTP " + std::to_string(status));
  std::string head = raw.substr(0, hdr_end);
  for (auto& c : head) c = static_cast<char>(tolower(c));
  const size_t ct = head.find("content-type:");
  if (ct != std::string::npos && content_type != nullptr) {
    size_t e = head.find("\r\n", ct);
    std::string v = head.substr(ct + 13, e == std::string::npos ? std::string::npos : e - ct - 13);
    while (!v.empty() && v.front() == ' ') v.erase(v.begin());
    *content_type = v;
  }
  std::string body = raw.substr(hdr_end + 4);
  if (head.find("transfer-encoding: chunked") != std::string::npos) {
    std::string out;
    size_t p = 0;
    while (p < body.size()) {
      const size_t eol = body.find("\r\n", p);
      if (eol == std::string::npos) break;
      const size_t len = strtoul(body.substr(p, eol - p).c_str(), nullptr, 16);
      if (len == 0) break;
      // the chunk length comes from the image host: it must fit in what was received, and the decoded
      // body obeys the same size limit as the raw response
      if (len > body.size() - (eol + 2)) throw std::runtime_error("malformed chunked image response");
      out.append(body, eol + 2, len);
      if (out.size() > max_bytes) throw std::runtime_error("image is larger than the size limit");
      p = eol + 2 + len + 2;
    }
    body.swap(out);
  }
  return body;
}

}  // namespace

std::optional<std::pair<uint32_t, uint32_t>> dimensions(const std::string& b, std::string* mimetype) {
  const unsigned char* p = reinterpret_cast<const unsigned char*>(b.data());
  const size_t n = b.size();
  auto mt = [&](const char* m) { if (mimetype != nullptr) *mimetype = m; };
  if (n >= 24 && memcmp(p, "\x89PNG\r\n\x1a\n", 8) == 0) {
    mt("image/png");
    return std::make_pair(be32(p + 16), be32(p + 20));
  }
  if (n >= 10 && (memcmp(p, "GIF87a", 6) == 0 || memcmp(p, "GIF89a", 6) == 0)) {
    mt("image/gif");
    return std::make_pair(le16(p + 6), le16(p + 8));
  }
  if (n >= 26 && p[0] == 'B' && p[1] == 'M') {
    mt("image/bmp");
    return std::make_pair(le32(p + 18), le32(p + 22));
  }
  if (n >= 30 && memcmp(p, "RIFF", 4) == 0 && memcmp(p + 8, "WEBP", 4) == 0) {
    mt("image/webp");
    if (memcmp(p + 12, "VP8 ", 4) == 0) return std::make_pair(le16(p + 26) & 0x3fff, le16(p + 28) & 0x3fff);
    if (memcmp(p + 12, "VP8L", 4) == 0) {
      const uint32_t v = le32(p + 21);
      return std::make_pair((v & 0x3fff) + 1, ((v >> 14) & 0x3fff) + 1);
    }
    if (memcmp(p + 12, "VP8X", 4) == 0)
      return std::make_pair((uint32_t(p[24]) | (uint32_t(p[25]) << 8) | (uint32_t(p[26]) << 16)) + 1,
                            (uint32_t(p[27]) | (uint32_t(p[28]) << 8) | (uint32_t(p[29]) << 16)) + 1);
    return std::nullopt;
  }
  if (n >= 4 && p[0] == 0xff && p[1] == 0xd8) {
    mt("image/jpeg");
    size_t i = 2;
    while (i + 9 < n) {
      if (p[i] != 0xff) {
        ++i;
        continue;
      }
      const unsigned char m = p[i + 1];
      if (m == 0xff) {
        ++i;
        continue;
      }
      if ((m >= 0xc0 && m <= 0xcf) && m != 0xc4 && m != 0xc8 && m != 0xcc)
        return std::make_pair(be16(p + i + 7), be16(p + i + 5));
      if (m == 0xd8 || m == 0x01 || (m >= 0xd0 && m <= 0xd7)) {
        i += 2;
        continue;
      }
      i += 2 + be16(p + i + 2);
    }
    return std::nullopt;
  }
  return std::nullopt;
}

Fetched fetch(const std::string& url, size_t max_bytes) {
  Fetched f;
  if (url.compare(0, 5, "data:") == 0) {
    const size_t comma = url.find(',');
    if (comma == std::string::npos) throw std::runtime_error("invalid image data URI");
    const std::string meta = url.substr(5, comma - 5);
    if (meta.find(";base64") == std::string::npos) throw std::runtime_error("image data URIs must be base64 encoded");
    f.mimetype = meta.substr(0, meta.find(';'));
    if ((url.size() - comma) * 3 / 4 > max_bytes) throw std::runtime_error("image is larger than the payload limit");
    f.data = base64_decode(url.substr(comma + 1));
  } else if (url.compare(0, 7, "http://") == 0) {
    f.data = http_get(url, max_bytes, &f.mimetype);
  } else if (url.compare(0, 8, "https://") == 0) {
    throw std::runtime_error("https image URLs are not supported by this router build: inline the image as a data: URI");
  } else {
    throw std::runtime_error("invalid image URL (expected data: or http://)");
  }
  if (f.data.empty()) throw std::runtime_error("empty image");
  if (f.data.size() > max_bytes) throw std::runtime_error("image is larger than the payload limit");
  std::string sniffed;
  auto dim = dimensions(f.data, &sniffed);
  if (!dim) throw std::runtime_error("unsupported image format (png, jpeg, gif, webp and bmp are recognised)");
  if (!sniffed.empty()) f.mimetype = sniffed;
  f.width = dim->first;
  f.height = dim->second;
  if (f.width == 0 || f.height == 0) throw std::runtime_error("image has a zero dimension");
  return f;
}

uint32_t tokens_per_image(const json::Value& config, uint32_t width, uint32_t height) {
  if (!config.is_object() || !config.has("vision_config")) return 0;
  const std::string mt = config.has("model_type") && config["model_type"].is_string() ? config["model_type"].as_string() : "";
  const json::Value& vis = config["vision_config"];
  auto num = [&](const char* k, double dflt) { return vis.is_object() && vis.has(k) ? vis[k].as_double() : dflt; };
  if (mt == "paligemma") {
    const uint32_t side = static_cast<uint32_t>(num("image_size", 224) / num("patch_size", 14));
    return side * side;
  }
  if (mt == "llava" || mt == "llava_next") {
    const uint32_t tile = static_cast<uint32_t>(num("image_size", 336));
    const uint32_t side = static_cast<uint32_t>(tile / num("patch_size", 14));
    if (mt == "llava" || !config.has("image_grid_pinpoints") || !config["image_grid_pinpoints"].is_array() ||
        width == 0 || height == 0)
      return side * side;   // one view: one feature row per patch
    // any-resolution tiling: base view + the tile map at the best-fitting resolution, without the rows / columns
    // that only saw padding, plus one newline per remaining row
    const double W = width, H = height;
    double best_h = 0, best_w = 0, best_eff = -1, best_waste = 1e300;
    for (const json::Value& pin : config["image_grid_pinpoints"].items()) {
      if (!pin.is_array() || pin.items().size() < 2) continue;
      const double h = pin.items()[0].as_double(), w = pin.items()[1].as_double();
      const double scale = std::min(w / W, h / H);
      const double eff = std::min(std::floor(W * scale) * std::floor(H * scale), W * H);
      const double waste = w * h - eff;
      if (eff > best_eff || (eff == best_eff && waste < best_waste)) {
        best_h = h; best_w = w; best_eff = eff; best_waste = waste;
      }
    }
    const long mh = static_cast<long>(best_h / tile) * side, mw = static_cast<long>(best_w / tile) * side;
    long rows = mh, cols = mw;
    if (W / H > static_cast<double>(mw) / mh) {
      const long new_h = static_cast<long>(std::nearbyint(H * (mw / W) * 1e7) / 1e7);
      rows = mh - 2 * ((mh - new_h) / 2);
    } else {
      const long new_w = static_cast<long>(std::nearbyint(W * (mh / H) * 1e7) / 1e7);
      cols = mw - 2 * ((mw - new_w) / 2);
    }
    return side * side + static_cast<uint32_t>(rows * (cols + 1));
  }
  if (mt == "qwen2_vl" || mt == "qwen2_5_vl") {
    // dynamic resolution: both sides rounded to multiples of patch * merge inside the pixel budget; one row
    // per merge x merge block of patches, plus the vision-start / vision-end tokens the runner adds
    const double patch = num("patch_size", 14), merge = num("spatial_merge_size", 2);
    const double factor = patch * merge;
    const double min_px = num("min_pixels", 56.0 * 56.0), max_px = num("max_pixels", 14.0 * 14.0 * 4.0 * 1280.0);
    // images at most 20 pixels wide are doubled before the resize, as the shard does
    const double H = width <= 20 ? 2.0 * height : height, W = width <= 20 ? 2.0 * width : width;
    double h = std::max(factor, std::nearbyint(H / factor) * factor);
    double w = std::max(factor, std::nearbyint(W / factor) * factor);
    if (h * w > max_px) {
      const double beta = std::sqrt(H * W / max_px);
      h = std::max(factor, std::floor(H / beta / factor) * factor);
      w = std::max(factor, std::floor(W / beta / factor) * factor);
    } else if (h * w < min_px) {
      const double beta = std::sqrt(min_px / (H * W));
      h = std::ceil(H * beta / factor) * factor;
      w = std::ceil(W * beta / factor) * factor;
    }
    uint32_t n = static_cast<uint32_t>((h / factor) * (w / factor));
    if (config.has("vision_start_token_id")) ++n;
    if (config.has("vision_end_token_id")) ++n;
    return n;
  }
  if (mt == "gemma3") {
    // fixed number of pooled rows per image, wrapped in begin-of-image / end-of-image tokens by the runner
    uint32_t n = config.has("mm_tokens_per_image") ? static_cast<uint32_t>(config["mm_tokens_per_image"].as_double()) : 256;
    if (config.has("boi_token_index") || config.has("boi_token_id")) ++n;
    if (config.has("eoi_token_index") || config.has("eoi_token_id")) ++n;
    // "\n\n" before the begin and after the end token when the tokenizer is a real one (`_gemma3.pad` tokens each side)
    if (config.has("_gemma3")) n += 2 * static_cast<uint32_t>(config["_gemma3"]["pad"].as_double());
    return n;
  }
  if (mt == "idefics") return 3;  // <fake_token_around_image><image><fake_token_around_image>; cross-attention carries the image
  if (mt == "mllama") return 1;   // one <|image|> token; the image itself reaches the text through cross-attention
  if (mt == "idefics2") {
    // perceiver resampler: a fixed number of latents per image
    const json::Value& pc = config.has("perceiver_config") ? config["perceiver_config"] : vis;
    const uint32_t seq =
        pc.is_object() && pc.has("resampler_n_latents") ? static_cast<uint32_t>(pc["resampler_n_latents"].as_double()) : 64;
    // `_idefics2` is added at start-up when the tokenizer has the marker token: the image's rows sit between markers,
    // and with image splitting the four quadrants come before the whole image (the shard's models/idefics2.py)
    if (!config.has("_idefics2")) return seq;
    const bool split = config["_idefics2"].has("split") && config["_idefics2"]["split"].as_bool() && width >= 2 && height >= 2;
    const uint32_t views = split ? 5 : 1;
    return views * (seq + 1) + 1;
  }
  if (mt == "idefics3") {
    // pixel shuffle folds scale x scale patches of a view into one row
    const uint32_t side = static_cast<uint32_t>(num("image_size", 364) / num("patch_size", 14));
    const uint32_t f = config.has("scale_factor") ? static_cast<uint32_t>(config["scale_factor"].as_double()) : 2;
    const uint32_t seq = f ? (side / f) * (side / f) : side * side;
    // Image splitting (the shard's models/idefics3.py does the same arithmetic): `_idefics3` is added to the config by
    // the router's start-up when the tokenizer has the marker tokens: {longest_edge, tile, split, nl, nlnl}
    if (!config.has("_idefics3") || width == 0 || height == 0) return seq;
    const json::Value& sp = config["_idefics3"];
    if (!sp.has("split") || !sp["split"].as_bool()) return seq + 3;
    const long tile = static_cast<long>(sp["tile"].as_double());
    const long longest = static_cast<long>(sp["longest_edge"].as_double());
    const uint32_t nl = static_cast<uint32_t>(sp["nl"].as_double()), nlnl = static_cast<uint32_t>(sp["nlnl"].as_double());
    long w, h;
    const double aspect = static_cast<double>(width) / static_cast<double>(height);
    if (width >= height) {
      w = longest;
      h = static_cast<long>(static_cast<double>(w) / aspect);
      h += h % 2;
    } else {
      h = longest;
      w = static_cast<long>(static_cast<double>(h) * aspect);
      w += w % 2;
    }
    h = std::max(h, 1L);
    w = std::max(w, 1L);
    const long upper = 4096;
    const double aspect2 = static_cast<double>(w) / static_cast<double>(h);
    if (w >= h && w > upper) {
      w = upper;
      h = static_cast<long>(static_cast<double>(w) / aspect2);
    } else if (h > w && h > upper) {
      h = upper;
      w = static_cast<long>(static_cast<double>(h) * aspect2);
    }
    h = std::max(h, 1L);
    w = std::max(w, 1L);
    const double aspect3 = static_cast<double>(w) / static_cast<double>(h);
    auto up = [tile](long v) { return (v + tile - 1) / tile * tile; };
    if (w >= h) {
      w = up(w);
      h = up(static_cast<long>(static_cast<double>(w) / aspect3));
    } else {
      h = up(h);
      w = up(static_cast<long>(static_cast<double>(h) * aspect3));
    }
    if (h <= tile && w <= tile) return seq + 3;      // one view between the markers
    const uint32_t rows = static_cast<uint32_t>(h / tile), cols = static_cast<uint32_t>(w / tile);
    return rows * cols * (seq + 2) + (rows - 1) * nl + nlnl + seq + 3;
  }
  return 0;
}

uint32_t placeholder_id(const std::string& data, uint32_t i) {
  uint64_t h = 1469598103934665603ull;   // FNV-1a over the image bytes
  for (unsigned char c : data) {
    h ^= c;
    h *= 1099511628211ull;
  }
  h ^= (static_cast<uint64_t>(i) + 0x9e3779b97f4a7c15ull) * 0xff51afd7ed558ccdull;
  return 0x80000000u | static_cast<uint32_t>((h ^ (h >> 32)) & 0x7fffffffu);
}

}  // namespace images
