// Housekeeping of a host's table images from outside a server: what lies under an image directory, which of it
// still belongs to a live node's current table, and removal of the rest.
//
// Parity: the reference keeps one persistent-memory pool per storage and cleans up with
// DCPmemory::remove_storage / remove_storage_exclude (pico-ps/storage/DCPmemory.cpp:169-210) and, for whole
// volumes that nothing mounts any more, scripts/clear_lvs.sh:3-20. Here an image is a file
// <dir>/node_<id>/storage_<sid>.img (written by Server::save_local_images), so the tool is a directory walk.
#pragma once
#include <dirent.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <fstream>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "../common/json.h"
#include "master.h"
#include "server.h"

namespace psb {

struct LocalImage {
    int node = -1;
    int32_t sid = -1;
    std::string path, uuid;
    uint32_t stride = 0;
    uint64_t records = 0, bytes = 0;
    bool readable = false;        // header intact and the file as long as the header says
    // with a master: "current" (a registered node's image of a table with this layout identity), "dead_node" (the
    // node is not registered: the image is what a server in restore mode would open), "stale" (the table is gone or
    // has another identity), "damaged"; without one: "unknown" or "damaged"
    std::string state = "unknown";
};

inline std::vector<std::string> image_dir_entries(const std::string& dir) {
    std::vector<std::string> out;
    if (DIR* d = ::opendir(dir.c_str())) {
        while (dirent* ent = ::readdir(d)) {
            const std::string name = ent->d_name;
            if (name != "." && name != "..") out.push_back(name);
        }
        ::closedir(d);
    }
    return out;
}

inline bool read_image_header(LocalImage* im) {
    std::ifstream f(im->path, std::ios::binary);
    char magic[8];
    uint64_t ulen = 0;
    f.read(magic, 8);
    f.read((char*)&ulen, 8);
    if (!f || std::memcmp(magic, "PSBIMG1", 8) != 0 || ulen > 4096) return false;
    im->uuid.assign(ulen, '\0');
    f.read(&im->uuid[0], (std::streamsize)ulen);
    f.read((char*)&im->stride, 4);
    f.read((char*)&im->records, 8);
    if (!f) return false;
    const uint64_t want = 8 + 8 + ulen + 4 + 8 + im->records * (8 + (uint64_t)im->stride * 4);
    return im->bytes == want;
}

// Every image under `dir`. With `master` each one is classified against the registry and the tables' contexts.
inline Status list_local_images(const std::string& dir, MasterClient* master, std::vector<LocalImage>* out) {
    out->clear();
    std::set<int> live;
    if (master) {
        std::map<int32_t, std::string> nodes;
        PSB_RETURN_IF_ERROR(master->get_nodes(PSERVER_S2S_RPC_NAME, &nodes));
        for (auto& kv : nodes) live.insert(kv.first);
    }
    std::map<int32_t, std::string> uuid_of;
    for (const std::string& node_dir : image_dir_entries(dir)) {
        if (node_dir.compare(0, 5, "node_") != 0) continue;
        for (const std::string& name : image_dir_entries(dir + "/" + node_dir)) {
            if (name.compare(0, 8, "storage_") != 0 || name.size() <= 12 || name.compare(name.size() - 4, 4, ".img") != 0) continue;
            LocalImage im;
            im.node = std::atoi(node_dir.c_str() + 5);
            im.sid = (int32_t)std::atoi(name.c_str() + 8);
            im.path = dir + "/" + node_dir + "/" + name;
            struct stat sb;
            if (::stat(im.path.c_str(), &sb) == 0) im.bytes = (uint64_t)sb.st_size;
            im.readable = read_image_header(&im);
            if (!im.readable) {
                im.state = "damaged";
            } else if (master) {
                if (!uuid_of.count(im.sid)) {
                    std::string json;
                    TableDescriptor td;
                    uuid_of[im.sid] = master->get_context(ctx_key(im.sid), &json).ok() && td.from_json_str(json) ? td.version_uuid : "";
                }
                if (uuid_of[im.sid].empty() || uuid_of[im.sid] != im.uuid) im.state = "stale";
                else im.state = live.count(im.node) ? "current" : "dead_node";
            }
            out->push_back(std::move(im));
        }
    }
    return Status::Ok();
}

// Remove the images that nobody can use any more: stale and damaged ones (and, with `dead_nodes_too`, those of
// nodes that are not registered - only when no server is going to be started in restore mode for them). Empty node
// directories go with them. Needs a master: without one nothing can be told apart.
inline Status remove_unused_local_images(const std::string& dir, MasterClient* master, bool dead_nodes_too, int* removed) {
    *removed = 0;
    if (!master) return Status::InvalidConfig("removing images needs the master to tell which are in use");
    std::vector<LocalImage> images;
    PSB_RETURN_IF_ERROR(list_local_images(dir, master, &images));
    for (const LocalImage& im : images) {
        const bool drop = im.state == "stale" || im.state == "damaged" || (dead_nodes_too && im.state == "dead_node");
        if (drop && ::unlink(im.path.c_str()) == 0) ++*removed;
    }
    for (const std::string& node_dir : image_dir_entries(dir))
        if (node_dir.compare(0, 5, "node_") == 0 && image_dir_entries(dir + "/" + node_dir).empty()) ::rmdir((dir + "/" + node_dir).c_str());
    return Status::Ok();
}

inline Json local_images_json(const std::vector<LocalImage>& images) {
    Json arr = Json::array();
    for (const LocalImage& im : images) {
        Json o = Json::object();
        o["node"] = (int64_t)im.node;
        o["storage_id"] = (int64_t)im.sid;
        o["path"] = im.path;
        o["version_uuid"] = im.uuid;
        o["stride"] = (int64_t)im.stride;
        o["records"] = (int64_t)im.records;
        o["bytes"] = (int64_t)im.bytes;
        o["state"] = im.state;
        arr.push_back(o);
    }
    return arr;
}

}  // namespace psb
